// The allocator step shared by the host builder (host_step.cu) and the device-resident one
// (device_step.cu): grow ONE request's page list in the reference's order — pages come from the
// prefetch buffer, which is refilled with the lowest free indices of the bitmap, at least
// fetch_size at a time (deserve_worker/kvcache/paged/page_pool.py:38-55, kvcache.py:21-29,
// virtual.py:138-149). One function compiled for both sides, so the page ids cannot differ.
#pragma once

#include <stdint.h>

#ifdef __CUDACC__
#define DSV_HD __host__ __device__
#else
#define DSV_HD
#endif

namespace dsv {

enum : int { GROW_OK = 0, GROW_NO_PAGES = 1, GROW_ROW_FULL = 2 };

// Grows the request whose table row is `row` (and flag row `isswap_row`, may be null) from
// *occupied pages to what want_tokens needs. Returns GROW_NO_PAGES (with *need = pages asked for)
// when the pool cannot give them, GROW_ROW_FULL when the row is too short; state is untouched then.
DSV_HD inline int grow_request(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int32_t buffer_cap,
                               int32_t* buffer_start, int32_t* buffer_len, int64_t* num_avails, int32_t fetch_size,
                               int32_t page_size, int32_t num_pages_main, int32_t* row, uint8_t* isswap_row,
                               int64_t table_cols, int want_tokens, int32_t* occupied, int32_t* need) {
  const int have = *occupied;
  if (want_tokens <= have * page_size) return GROW_OK;
  const int new_n = (want_tokens + page_size - 1) / page_size;
  const int size = new_n - have;
  *need = new_n;
  if (new_n > table_cols) return GROW_ROW_FULL;
  *need = size;
  if (size > *num_avails) return GROW_NO_PAGES;  // the reference's ValueError("Not enough pages")
  *num_avails -= size;
  if (size > *buffer_len) {  // refill: the lowest free indices, at least fetch_size of them
    const int short_by = size - *buffer_len;
    const int want = fetch_size > short_by ? fetch_size : short_by;
    if (*buffer_start + *buffer_len + want > buffer_cap) {  // compact the window to the front
      for (int k = 0; k < *buffer_len; ++k) buffer[k] = buffer[*buffer_start + k];
      *buffer_start = 0;
    }
    int32_t* tail = buffer + *buffer_start + *buffer_len;
    int got = 0;
    for (int pg = 0; pg < num_pages && got < want; ++pg)
      if (bitmap[pg]) {
        bitmap[pg] = 0;
        tail[got++] = pg;
      }
    *buffer_len += got;
  }
  const int32_t* ids = buffer + *buffer_start;
  for (int k = 0; k < size; ++k) {
    row[have + k] = ids[k];
    if (isswap_row != nullptr) isswap_row[have + k] = ids[k] >= num_pages_main ? 1 : 0;
  }
  *buffer_start += size;
  *buffer_len -= size;
  *occupied = new_n;
  return GROW_OK;
}

}  // namespace dsv
