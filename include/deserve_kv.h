/*
 * deserve_kv.h — C ABI of libdeserve_kv.so: the paged KV-cache hot path of
 * DeServe (CoLearn-Dev/deserve) as hand-written sm_100a CUDA kernels.
 *
 * Every entry point
 *   - takes plain pointers, sizes and a CUDA stream passed as void* (a
 *     cudaStream_t; NULL = the legacy default stream),
 *   - validates its arguments BEFORE launching anything,
 *   - returns 0 on success or a negative DSV_E_* code (never throws, never
 *     exits); dsv_last_error() gives the message of the calling thread's
 *     last failure,
 *   - is stream-ordered and does not synchronise unless its comment says so,
 *   - allocates nothing: all buffers belong to the caller.
 *
 * Page tensor layout (kept from the reference, deserve_worker/kvcache/paged/
 * page_pool.py:25-29): pages[L, P, 2, page_size, n_kv_heads, head_dim], index
 * 2 = {0: K, 1: V}. Kernels receive one layer's slab, pages[layer]
 * (page_pool.py:81-82), plus the page stride in ELEMENTS
 * (= 2 * page_size * n_kv_heads * head_dim for a contiguous pool).
 *
 * Ragged-batch descriptors (deserve_worker/model/context/flash.py:24-70), all
 * int32 on the device:
 *   qo_indptr[B+1]        prefix sum of new tokens per request
 *   kv_indices[sum pages] page ids of every request, concatenated
 *   kv_indptr[B+1]        prefix sum of pages per request
 *   kv_last_page_len[B]   valid tokens in each request's last page (1..page_size)
 * and they describe the cache AFTER the step's new tokens were appended.
 */
#ifndef DESERVE_KV_H_
#define DESERVE_KV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSV_VERSION 100

/* element types of K/V pages, q and out */
#define DSV_F32 0
#define DSV_F16 1
#define DSV_BF16 2

/* error codes */
#define DSV_OK 0
#define DSV_E_INVALID (-1)     /* bad argument (null pointer, size, alignment, unsupported shape) */
#define DSV_E_CUDA (-2)        /* a CUDA runtime call failed; message holds cudaGetErrorString */
#define DSV_E_WORKSPACE (-3)   /* caller's workspace / plan buffer too small */
#define DSV_E_UNSUPPORTED (-4) /* valid request that this build has no kernel for */
#define DSV_E_DEVICE (-5)      /* a kernel reported a failed bounds check or a wait that gave up */

/* Library version (DSV_VERSION of the build). */
int dsv_version(void);

/* Message of the calling thread's last error ("" if none). Never NULL. */
const char* dsv_last_error(void);

/* SM count and compute capability of the current CUDA device. Synchronous, cheap. */
int dsv_device_info(int* sm_count, int* cc_major, int* cc_minor);

/*
 * Append-scatter of one step's new K/V rows into one layer's pages.
 * Replaces the call flashinfer.append_paged_kv_cache(xk, xv, indptr, pages,
 * kv_page_indices, kv_page_indptr, kv_last_page_lens) at
 * deserve_worker/model/layer/attention.py:174-183.
 * Request i has n_i = qo_indptr[i+1]-qo_indptr[i] new tokens and post-append
 * length len_i = (kv_indptr[i+1]-kv_indptr[i]-1)*page_size + kv_last_page_len[i];
 * new token j goes to position t = len_i - n_i + j, i.e. page
 * kv_indices[kv_indptr[i] + t / page_size], slot t % page_size.
 * k, v: [nnz, n_kv_heads, head_dim] with a token stride in elements
 * (heads and dims contiguous). num_pages: pages in the layer slab; a page id
 * outside [0, num_pages) is skipped and recorded in the device status word.
 * Pure data movement: bit-exact.
 */
int dsv_append_paged_kv(const void* k, const void* v, int64_t k_stride_tok, int64_t v_stride_tok,
                        const int32_t* qo_indptr, void* pages_layer, int64_t page_stride,
                        int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                        const int32_t* kv_last_page_len, int batch, int nnz, int n_kv_heads,
                        int head_dim, int page_size, int dtype, void* stream);

/*
 * Interleaved-pair rotary embedding applied in place to ragged q and k, the
 * position of token j of request i being offsets[i] + j. Replaces
 * flashinfer.apply_rope(xq, xk, indptr, offsets, interleave=True,
 * rope_theta=...) at deserve_worker/model/layer/attention.py:166-173 (torch
 * statement of the same rotation: attention.py:45-72 with the table of
 * deserve_worker/execution/exec.py:25-55). Angles and the rotation are
 * computed in fp32 and rounded once to the tensor type. inv_freq_host
 * (optional, HOST memory, head_dim/2 floats) overrides the frequency table
 * theta^(-2i/head_dim), e.g. with the table torch computed, so that the angles
 * match a torch reference bit for bit; NULL derives it from rope_theta.
 */
int dsv_apply_rope_inplace(void* q, void* k, int64_t q_stride_tok, int64_t k_stride_tok,
                           const int32_t* qo_indptr, const int32_t* offsets, int batch, int nnz,
                           int n_q_heads, int n_kv_heads, int head_dim, float rope_theta,
                           const float* inv_freq_host, int dtype, void* stream);

/*
 * Rotary embedding fused into the append-scatter: q is rotated in place, k is
 * rotated and written straight into its page slot, v is copied into its page
 * slot (k itself is left untouched). One launch instead of the reference's
 * apply_rope + append_paged_kv_cache pair (deserve_worker/model/layer/
 * attention.py:166-183); the rotation is the same fp32 expression as
 * dsv_apply_rope_inplace, so pages and q agree with that pair bit for bit.
 */
int dsv_rope_append_paged_kv(void* q, const void* k, const void* v, int64_t q_stride_tok,
                             int64_t k_stride_tok, int64_t v_stride_tok,
                             const int32_t* qo_indptr, const int32_t* offsets, void* pages_layer,
                             int64_t page_stride, int64_t num_pages, const int32_t* kv_indices,
                             const int32_t* kv_indptr, const int32_t* kv_last_page_len, int batch,
                             int nnz, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                             float rope_theta, const float* inv_freq_host, int dtype,
                             void* stream);

/*
 * out[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * weight, fp32 math, rounded
 * once. Replaces flashinfer.norm.rmsnorm(x, weight, eps) at
 * deserve_worker/model/layer/norm.py:34 (torch statement: norm.py:18-19, 37-39).
 * Row strides in elements; out may alias x.
 */
int dsv_rmsnorm(const void* x, const void* weight, void* out, int64_t x_stride,
                int64_t out_stride, int rows, int dim, float eps, int dtype, void* stream);

/*
 * out[r, c] = silu(gate_up[r, c]) * gate_up[r, ffn_dim + c] for c in [0, ffn_dim): the
 * elementwise middle of the SwiGLU feed-forward, F.silu(self.w1(x)) * self.w3(x) at
 * deserve_worker/model/layer/linear.py:121-123, on the output of ONE projection whose
 * rows hold the gate columns followed by the up columns (w1 and w3 stacked). fp32 math;
 * silu is rounded to dtype and so is the product, like the two torch statements. Row
 * strides in elements.
 */
int dsv_silu_mul(const void* gate_up, void* out, int64_t gate_up_stride, int64_t out_stride,
                 int rows, int ffn_dim, int dtype, void* stream);

/*
 * Greedy sampling: tokens[r] = argmax of logits[r, 0..vocab), the lowest index
 * among equal maxima. Replaces the per-task torch.argmax + torch.cat loop of
 * deserve_worker/layer_storage.py:219-253 (temperature 0 branch, line 250).
 */
int dsv_greedy_sample(const void* logits, int64_t row_stride, int rows, int vocab,
                      int32_t* tokens, int dtype, void* stream);

/*
 * Host-side planning of the split-KV schedule for paged decode attention.
 * Replaces BatchDecodeWithPagedKVCacheWrapper.begin_forward(...) at
 * deserve_worker/execution/exec.py:184-192. Pure host arithmetic: reads
 * kv_indptr_host[batch+1] (HOST memory), writes an int32 plan into plan_host
 * (HOST memory, plan_capacity_i32 entries available) and reports how many
 * entries it used and how many bytes of device workspace dsv_paged_decode
 * needs for that plan. The caller copies plan_host[0..used) to the device.
 * sm_count: SMs to balance for (dsv_device_info); <= 0 means 148.
 */
int dsv_decode_plan(const int32_t* kv_indptr_host, int batch, int n_q_heads, int n_kv_heads,
                    int head_dim, int page_size, int dtype, int sm_count, int32_t* plan_host,
                    int64_t plan_capacity_i32, int64_t* plan_used_i32,
                    int64_t* workspace_bytes);

/*
 * Batched paged GQA decode attention over one layer's pages:
 *   out[i,h,:] = sum_t softmax_t(q[i,h] . K[i,t,h/G] * sm_scale) * V[i,t,h/G],
 * t in [0, len_i), G = n_q_heads / n_kv_heads, no mask, no positional term,
 * fp32 softmax and accumulation, output rounded once to dtype. Replaces
 * BatchDecodeWithPagedKVCacheWrapper.forward(xq, pages) at
 * deserve_worker/model/layer/attention.py:185 (plan/end_forward:
 * deserve_worker/execution/exec.py:184-198).
 * q, out: [batch, n_q_heads, head_dim], token stride in elements.
 * plan_host / plan_dev: the same plan on the host (header is read there) and
 * on the device. workspace: device scratch of at least the size the plan
 * reported (may be NULL when that size is 0). lse (optional, may be NULL):
 * [batch, n_q_heads] natural-log sum-exp of the scaled scores. num_pages:
 * pages in the layer slab (bound of the page ids and of the TMA tensor map).
 * Kernel choice: 16-bit K/V, GQA group <= 16, power-of-two page size >= 8 and
 * a dense pool (page_stride = one page) run the TMA + tensor-core kernel;
 * other 16-bit shapes the cp.async + tensor-core kernel; fp32 (and GQA groups
 * above 16) the CUDA-core kernel.
 */
int dsv_paged_decode(const void* q, int64_t q_stride_tok, const void* pages_layer,
                     int64_t page_stride, int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                     const int32_t* kv_last_page_len, void* out, int64_t out_stride_tok,
                     float* lse, const int32_t* plan_host, const int32_t* plan_dev,
                     void* workspace, int64_t workspace_bytes, int batch, int n_q_heads,
                     int n_kv_heads, int head_dim, int page_size, int dtype, float sm_scale,
                     void* stream);

/*
 * Host-side planning for ragged causal paged prefill attention. Replaces
 * BatchPrefillWithPagedKVCacheWrapper.begin_forward(...) at
 * deserve_worker/execution/exec.py:227-236. Reads qo_indptr_host[batch+1] and
 * kv_len_host[batch] (HOST memory; kv_len = post-append length of each
 * request) and writes the list of (request, q-tile) work items: a tile holds
 * 128 / (n_q_heads / n_kv_heads) q tokens and knows how many kv positions its
 * last token sees (all of them when causal = 0). Requests with fewer than
 * min_new_tokens new tokens get no work item (a caller that sends the decode
 * rows of a mixed batch to dsv_paged_decode passes 2). Pure host arithmetic.
 * The plan is opaque to the caller: a 12-integer header, then the items (four
 * integers each) of the single-CTA kernel and those of the two-CTA kernel; the
 * latter list is empty unless the environment holds DESERVE_PREFILL_PAIRS=1
 * (head_dim 128, pages of 16 tokens or more). Items run the longest request
 * first, a request's items together.
 */
int dsv_prefill_plan(const int32_t* qo_indptr_host, const int32_t* kv_len_host, int batch,
                     int n_q_heads, int n_kv_heads, int head_dim, int page_size, int dtype,
                     int causal, int min_new_tokens, int32_t* plan_host,
                     int64_t plan_capacity_i32, int64_t* plan_used_i32);

/*
 * Ragged causal attention of nnz new q rows against paged K/V (chunked
 * prefill, and mixed prefill+decode batches) on the tcgen05 tensor cores. q
 * row j (of n_i) of request i sees kv positions <= len_i - n_i + j (all
 * positions when causal = 0). Replaces
 * BatchPrefillWithPagedKVCacheWrapper.forward(xq, pages, causal=True) at
 * deserve_worker/model/layer/attention.py:188-192. fp16 / bf16 only
 * (DSV_E_UNSUPPORTED for fp32), head_dim 64 or 128, power-of-two page size,
 * dense pool, GQA group dividing 128. fp32 softmax and accumulation; P is
 * rounded to the 16-bit type before P.V, the output once at the end.
 */
int dsv_paged_prefill(const void* q, int64_t q_stride_tok, const int32_t* qo_indptr,
                      const void* pages_layer, int64_t page_stride, int64_t num_pages,
                      const int32_t* kv_indices, const int32_t* kv_indptr,
                      const int32_t* kv_last_page_len, void* out, int64_t out_stride_tok,
                      const int32_t* plan_host, const int32_t* plan_dev, int batch, int nnz,
                      int n_q_heads, int n_kv_heads, int head_dim, int page_size, int dtype,
                      float sm_scale, int causal, void* stream);

/*
 * dsv_paged_decode for callers that cannot allocate device memory. It has no
 * counterpart in the reference. Same arguments and results as dsv_paged_decode,
 * minus the workspace: the split-KV partial states live in a fixed scratch
 * array inside the library (DSV_STATIC_SCRATCH_BYTES, held by every GPU that
 * loads the library until the process exits). Meant for hosts that bind this C
 * ABI directly and have no device allocator left to ask: a serving worker that
 * gave all remaining HBM to the page pool at start-up, so a later cudaMalloc
 * fails or forces the pool to shrink; or a decode loop that cannot afford the
 * device-wide synchronisation a cudaMalloc / cudaFree implies.
 *  - The call allocates nothing (no cudaMalloc/cudaFree, no library allocator).
 *  - A plan whose partial states need more than DSV_STATIC_SCRATCH_BYTES is
 *    rejected with DSV_E_WORKSPACE before anything is launched.
 *  - The first call on each device resolves the scratch array's device address
 *    (with that device current); make that first call before any stream
 *    capture begins.
 *  - All calls on a device share the one array. Nothing in it has to start at
 *    zero (every partial state is written before it is read within a call), but
 *    two calls that overlap on the GPU (different streams) race on it:
 *    serialise them.
 */
#define DSV_STATIC_SCRATCH_BYTES (16 << 20)
int dsv_paged_decode_static(const void* q, int64_t q_stride_tok, const void* pages_layer,
                            int64_t page_stride, int64_t num_pages, const int32_t* kv_indices,
                            const int32_t* kv_indptr, const int32_t* kv_last_page_len, void* out,
                            int64_t out_stride_tok, float* lse, const int32_t* plan_host,
                            const int32_t* plan_dev, int batch, int n_q_heads, int n_kv_heads,
                            int head_dim, int page_size, int dtype, float sm_scale, void* stream);

/*
 * Gather scattered pages of several tasks into one dense buffer (pack), or
 * scatter such a buffer back into pages (unpack), for the layer window
 * [layer_begin, layer_end). Task t owns page ids
 * page_ids[ids_indptr[t] .. ids_indptr[t+1]) (n_t of them; ids_indptr[0] = 0).
 * In the packed buffer the tasks follow one another, task t starting at row
 * ids_indptr[t] * (layer_end - layer_begin), and inside a task the rows are
 * LAYER-MAJOR: row (l - layer_begin) * n_t + p holds pages[l, id_p]
 * (page_bytes each). That is the chunk layout of
 * KVCacheManager.copy_gpu_to_cpu / copy_cpu_to_gpu
 * (deserve_worker/kvcache/manager.py:38-44, 63-73). page_ids and ids_indptr
 * (n_tasks+1 entries) are DEVICE arrays. num_pages: pages in a layer slab
 * (layer_stride_bytes >= num_pages * page_bytes is checked on the host); a page
 * id outside [0, num_pages) is skipped — nothing is read or written for that
 * row — and recorded in the device status word. Bit-exact.
 */
int dsv_pack_pages(const void* pages_base, int64_t layer_stride_bytes, int64_t page_bytes,
                   int64_t num_pages, const int32_t* page_ids, const int32_t* ids_indptr,
                   int n_tasks, int64_t total_ids, int layer_begin, int layer_end, void* dst,
                   void* stream);
int dsv_unpack_pages(const void* src, void* pages_base, int64_t layer_stride_bytes,
                     int64_t page_bytes, int64_t num_pages, const int32_t* page_ids,
                     const int32_t* ids_indptr, int n_tasks, int64_t total_ids, int layer_begin,
                     int layer_end, void* stream);

/*
 * Per-task offload (swap-out) and reload (swap-in) between scattered HBM pages
 * and per-task chunks of a pinned host pool, through a device staging buffer:
 * pack kernel -> large cudaMemcpyAsync bursts, or bursts -> unpack kernel,
 * one layer window at a time, double-buffered over the two halves of
 * `staging` so that the DMA of one window overlaps the pack/unpack of the
 * next. Kernels run on stream_kernel, DMA on stream_dma; `events` are 4
 * cudaEvent_t of the caller (timing disabled). Replaces the advanced-index
 * gather + blocking copy_ of deserve_worker/kvcache/manager.py:24-46 and the
 * .to("cuda") + index_put of manager.py:48-86. Task t's chunk starts at
 * host_pool + chunk_row_begin_host[t] * page_bytes and holds
 * num_layers * n_t rows, layer-major. ids_indptr_host is the HOST copy of
 * ids_indptr. Half of the staging buffer must hold one layer of all tasks
 * (total_ids * page_bytes) or the call fails with DSV_E_WORKSPACE. num_pages
 * bounds the page ids as in dsv_pack_pages.
 * Asynchronous: the caller waits on both streams (swap-out: host data valid
 * after stream_dma; swap-in: pages valid after stream_kernel). Calls that share
 * `staging` may follow one another without a host wait as long as they also
 * share the two streams and the four events: every window first waits for the
 * event that marks the last use of its staging half, whichever call recorded it.
 */
int dsv_swap_out_pages(const void* pages_base, int64_t layer_stride_bytes, int64_t page_bytes,
                       int64_t num_pages, int num_layers, const int32_t* page_ids,
                       const int32_t* ids_indptr, const int32_t* ids_indptr_host,
                       const int64_t* chunk_row_begin_host, int n_tasks, void* staging,
                       int64_t staging_bytes, void* host_pool, void* stream_kernel,
                       void* stream_dma, void** events);
int dsv_swap_in_pages(const void* host_pool, void* pages_base, int64_t layer_stride_bytes,
                      int64_t page_bytes, int64_t num_pages, int num_layers,
                      const int32_t* page_ids, const int32_t* ids_indptr,
                      const int32_t* ids_indptr_host, const int64_t* chunk_row_begin_host,
                      int n_tasks, void* staging, int64_t staging_bytes, void* stream_kernel,
                      void* stream_dma, void** events);

/*
 * Microbatch region swap: for every layer l, copy the first out_bytes of the slab
 * pages_base + l*layer_stride_bytes + region_offset_bytes (the region is
 * region_bytes long, contiguous) to host_out + l*region_bytes, then fill the
 * first in_bytes of the same slab from host_in + l*region_bytes. out_bytes =
 * in_bytes = region_bytes moves the whole region, which is the data movement
 * VirtualPagePool.swap() states in torch (deserve_worker/kvcache/virtual.py:97-113)
 * and that swap.swap(d, h0, h1, s0, s1, interval)
 * (deserve_worker/kvcache/swap.cpp:9-57, called from virtual.py:79-95) is meant
 * to perform. Smaller values move only the head of the region: the allocator
 * hands out the lowest free page first, so the pages in use sit at the head and a
 * caller that knows the highest page in use (from the region's bitmap) need not
 * move the free tail. All outgoing copies run on stream_out in layer order; the
 * incoming copy of a group of layers runs on stream_in once that group's outgoing
 * copy has finished (`event`, a cudaEvent_t of the caller, carries the edge), so
 * both directions of the host link are busy at once. host_out or host_in may be
 * NULL to skip that direction. Bit-exact. Asynchronous: wait on both streams.
 * A page is [K: page_size token rows][V: page_size token rows]; out_rows /
 * in_rows < page_size move only the first rows of every half of the travelling
 * pages (for a caller that knows that no page of the head holds more tokens:
 * the tail pages of sequences that grow a token per step), as a 2-D copy that
 * keeps the region's layout in the host image. page_bytes = 0 or rows =
 * page_size: whole pages.
 */
int dsv_region_swap(void* pages_base, int num_layers, int64_t layer_stride_bytes,
                    int64_t region_offset_bytes, int64_t region_bytes, int64_t out_bytes,
                    int64_t in_bytes, void* host_out, const void* host_in, void* stream_out,
                    void* stream_in, void* event, int64_t page_bytes, int32_t page_size,
                    int32_t out_rows, int32_t in_rows);

/*
 * The host half of a step in one native call (no CUDA): for every request of
 * the batch, grow its page list to max(start_pos + seqlen, initial_seqlen)
 * tokens — pages come from the prefetch buffer, refilled with the lowest free
 * indices, at least fetch_size at a time, exactly the reference's order
 * (deserve_worker/kvcache/paged/page_pool.py:38-55, kvcache.py:21-29,
 * virtual.py:138-149) — then write the ragged-batch descriptors of
 * deserve_worker/model/context/flash.py:29-64 into `out` as six 4-int32-aligned
 * sections: indptr, kv_page_indptr, kv_last_page_lens, offsets, seqlens,
 * kv_page_indices (section_offsets[0..6], the last entry = int32 used).
 * All arrays are caller-owned HOST memory: bitmap[num_pages] (1 = free),
 * buffer[buffer_cap >= num_pages] with the live window (buffer_start,
 * buffer_len), tables[max_requests, table_cols] and the optional isswap flags
 * of the same shape (page id >= num_pages_main), slot / occupied per request.
 * When a request needs more pages than are available the call stops there and
 * returns DSV_E_WORKSPACE with failed_request / failed_need set (the
 * reference's ValueError("Not enough pages")); earlier requests stay grown.
 */
int dsv_host_build_step(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int32_t buffer_cap,
                        int32_t* buffer_start, int32_t* buffer_len, int64_t* num_avails,
                        int32_t fetch_size, int32_t page_size, int32_t num_pages_main,
                        int32_t* tables, uint8_t* isswap, int64_t table_cols, int batch,
                        const int32_t* slot, int32_t* occupied, const int32_t* start_pos,
                        const int32_t* seqlen, const int32_t* initial_seqlen, int32_t* out,
                        int64_t out_capacity, int64_t* section_offsets, int32_t* failed_request,
                        int32_t* failed_need);

/*
 * The same step with the allocator state on the DEVICE: bitmap[num_pages] (1 = free),
 * buffer[num_pages] (prefetched free ids), state (int64[2]: free pages; then the
 * prefetch window as two int32, start and length), tables[max_requests, table_cols]
 * and occupied[max_requests] (pages per table row) are device arrays that only these
 * kernels touch. req is a DEVICE array of batch x 6 int32 per request: table row,
 * start_pos, seqlen, initial_seqlen, and the two prefix sums the host can compute
 * from token counts alone (first new-token row, first page-list entry). With grow = 1
 * one thread first grows the requests in batch order with the very function the host
 * builder uses (same page ids as deserve_worker/kvcache/paged/page_pool.py:38-55 hands
 * out); then one CTA per request writes the six descriptor sections of
 * deserve_worker/model/context/flash.py:29-64 into `out` (device) at
 * section_offsets_host[0..6) (HOST array, same order as dsv_host_build_step), page
 * ids copied straight from the table rows. The caller checks the page budget and the
 * row length on its own counters before the call (it raises the reference's
 * ValueError itself); a disagreement shows up in the device status word.
 * dsv_device_free_rows returns the pages of the given table rows (device array of n
 * row numbers) to the bitmap and empties the rows (PagedKVCache.free,
 * kvcache.py:31-33; page_pool.py:73-76).
 */
int dsv_device_build_step(uint8_t* bitmap, int32_t num_pages, int32_t* buffer, int64_t* state,
                          int32_t fetch_size, int32_t page_size, int32_t* tables,
                          int64_t table_cols, int32_t* occupied, int32_t max_requests,
                          const int32_t* req, int batch, int grow, int32_t* out,
                          const int64_t* section_offsets_host, void* stream);
int dsv_device_free_rows(uint8_t* bitmap, int32_t num_pages, int64_t* state, const int32_t* tables,
                         int64_t table_cols, int32_t* occupied, const int32_t* slots, int n,
                         void* stream);

/*
 * The hop between pipeline stages over peer memory. The reference posts each
 * microbatch's activations to the next worker over HTTP
 * (deserve_worker/engine/pipeline/processor.py:218-224, PipelineProcessor.send_request);
 * on one NVLink node the sender stores them into the next GPU's inbox instead.
 *   dsv_peer_push   copies `bytes` (multiple of 16) from src (local) to dst (a
 *                   peer-mapped or local device address) with plain 16-byte stores and,
 *                   when every store is visible system-wide, writes `value` to *flag
 *                   (normally in the receiver's memory). `arrivals`: one uint32 of local
 *                   device scratch, zero before the first call (it returns to zero).
 *   dsv_peer_signal writes `value` to *flag after a system-wide fence (credits going back
 *                   to the sender).
 *   dsv_peer_wait   holds the stream until *flag >= value: one thread polls with
 *                   acquire loads for at most timeout_ns nanoseconds of the GPU's global
 *                   timer; on expiry the kernel ends, the device status reads 4 (wait
 *                   timeout) and the stream continues.
 * Flags are int32 that only grow (message number + 1). No TMA, no multicast: peer
 * memory is written with ordinary stores only. While the status word holds a wait
 * timeout, later pushes, signals and waits of the process do nothing (a link that lost a
 * message must not credit or overwrite buffers); dsv_read_device_status reports and
 * clears it.
 */
int dsv_peer_push(void* dst, const void* src, int64_t bytes, int32_t* flag, int32_t value,
                  uint32_t* arrivals, int sm_count, void* stream);
int dsv_peer_signal(int32_t* flag, int32_t value, void* stream);
int dsv_peer_wait(const int32_t* flag, int32_t value, int64_t timeout_ns, void* stream);

/*
 * Self-test of the bounded waits every mbarrier-based kernel here uses: launches
 * one thread that polls (at most `polls` times) a barrier phase nothing will
 * ever complete. The wait gives up, the kernel ends normally and
 * dsv_read_device_status then reports 4 (wait timeout); the context stays
 * usable. No counterpart in the reference (its kernels are third-party).
 */
int dsv_selftest_wait_timeout(int polls, void* stream);

/*
 * Device status word of the kernels' self-checks (page id / slot / token
 * bounds, bounded waits). Synchronises the device. *status = 0 when nothing
 * was recorded; otherwise a DSV_E_DEVICE detail code, cleared by the call.
 */
int dsv_read_device_status(int* status);

#ifdef __cplusplus
}
#endif
#endif /* DESERVE_KV_H_ */
