// Append-scatter of new K/V rows into pages, and in-place rotary embedding of
// ragged q/k. Both are pure streaming kernels: one 16-byte vector per thread,
// consecutive threads on consecutive vectors of a token row.
#include "common.cuh"

namespace dsv {
namespace {

// Request that owns ragged row `tok`: largest i with indptr[i] <= tok.
__device__ __forceinline__ int find_request(const int32_t* __restrict__ indptr, int batch, int tok) {
  int lo = 0, hi = batch;  // invariant: indptr[lo] <= tok < indptr[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (__ldg(indptr + mid) <= tok) lo = mid; else hi = mid;
  }
  return lo;
}

// One thread moves one 16-byte vector of K or of V.
// vec index -> (token, kv half, vector inside the Hkv*D row).
__global__ void __launch_bounds__(256)
append_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, int64_t k_stride_vec,
              int64_t v_stride_vec, const int32_t* __restrict__ qo_indptr, uint4* __restrict__ pages,
              int64_t page_stride_vec, int64_t num_pages, const int32_t* __restrict__ kv_indices,
              const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_last_page_len,
              int batch, int nnz, int row_vecs, int page_size, int* status) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)nnz * 2 * row_vecs;
  if (gid >= total) return;
  const int vec = (int)(gid % row_vecs);
  const int half = (int)((gid / row_vecs) & 1);
  const int tok = (int)(gid / (2 * row_vecs));

  const int req = find_request(qo_indptr, batch, tok);
  const int q0 = __ldg(qo_indptr + req), q1 = __ldg(qo_indptr + req + 1);
  const int p0 = __ldg(kv_indptr + req), p1 = __ldg(kv_indptr + req + 1);
  if (tok < q0 || tok >= q1 || p1 <= p0) {
    record_status(status, ST_BAD_REQUEST);
    return;
  }
  const int kv_len = (p1 - p0 - 1) * page_size + __ldg(kv_last_page_len + req);
  const int pos = kv_len - (q1 - q0) + (tok - q0);
  if (pos < 0) {
    record_status(status, ST_BAD_REQUEST);
    return;
  }
  const int page = __ldg(kv_indices + p0 + pos / page_size);
  const int slot = pos % page_size;
  if (page < 0 || page >= num_pages) {
    record_status(status, ST_BAD_PAGE_ID);
    return;
  }
  const uint4* src = half == 0 ? k + (int64_t)tok * k_stride_vec : v + (int64_t)tok * v_stride_vec;
  uint4* dst = pages + (int64_t)page * page_stride_vec +
               ((int64_t)half * page_size + slot) * row_vecs;
  dst[vec] = __ldg(src + vec);
}

struct RopeTable {
  float inv_freq[128];  // head_dim / 2 entries used (head_dim <= 256)
};

// One thread owns one (token, pair) and walks all q and k heads with the same
// cos/sin. Pairs are adjacent elements (2i, 2i+1) — the "interleaved" layout.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(T* __restrict__ q, T* __restrict__ k, int64_t q_stride, int64_t k_stride,
            const int32_t* __restrict__ qo_indptr, const int32_t* __restrict__ offsets, int batch,
            int nnz, int n_q_heads, int n_kv_heads, int head_dim, RopeTable table, int* status) {
  const int half_dim = head_dim >> 1;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (int64_t)nnz * half_dim) return;
  const int pair = (int)(gid % half_dim);
  const int tok = (int)(gid / half_dim);
  const int req = find_request(qo_indptr, batch, tok);
  const int q0 = __ldg(qo_indptr + req);
  if (tok < q0 || tok >= __ldg(qo_indptr + req + 1)) {
    record_status(status, ST_BAD_REQUEST);
    return;
  }
  const float pos = (float)(__ldg(offsets + req) + (tok - q0));
  const float angle = pos * table.inv_freq[pair];
  float sn, cs;
  sincosf(angle, &sn, &cs);
  T* qrow = q + (int64_t)tok * q_stride + 2 * pair;
  for (int h = 0; h < n_q_heads; ++h) {
    const float a = to_f32(qrow[0]), b = to_f32(qrow[1]);
    qrow[0] = from_f32<T>(a * cs - b * sn);
    qrow[1] = from_f32<T>(a * sn + b * cs);
    qrow += head_dim;
  }
  T* krow = k + (int64_t)tok * k_stride + 2 * pair;
  for (int h = 0; h < n_kv_heads; ++h) {
    const float a = to_f32(krow[0]), b = to_f32(krow[1]);
    krow[0] = from_f32<T>(a * cs - b * sn);
    krow[1] = from_f32<T>(a * sn + b * cs);
    krow += head_dim;
  }
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_append_paged_kv(const void* k, const void* v, int64_t k_stride_tok, int64_t v_stride_tok,
                        const int32_t* qo_indptr, void* pages_layer, int64_t page_stride,
                        int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                        const int32_t* kv_last_page_len, int batch, int nnz, int n_kv_heads,
                        int head_dim, int page_size, int dtype, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "append: unknown dtype %d", dtype);
  DSV_REQUIRE(batch >= 0 && nnz >= 0, "append: negative batch (%d) or nnz (%d)", batch, nnz);
  if (batch == 0 || nnz == 0) return DSV_OK;
  DSV_REQUIRE(k && v && qo_indptr && pages_layer && kv_indices && kv_indptr && kv_last_page_len,
              "append: null pointer argument");
  DSV_REQUIRE(n_kv_heads > 0 && head_dim > 0 && page_size > 0 && num_pages > 0, "append: non-positive shape");
  const int es = elem_size(dtype);
  const int64_t row_bytes = (int64_t)n_kv_heads * head_dim * es;
  DSV_REQUIRE(row_bytes % 16 == 0, "append: n_kv_heads*head_dim*elem_size (%lld) not a multiple of 16",
              (long long)row_bytes);
  DSV_REQUIRE(k_stride_tok >= (int64_t)n_kv_heads * head_dim && v_stride_tok >= (int64_t)n_kv_heads * head_dim,
              "append: token stride smaller than a row");
  DSV_REQUIRE((k_stride_tok * es) % 16 == 0 && (v_stride_tok * es) % 16 == 0 && (page_stride * es) % 16 == 0,
              "append: strides must be multiples of 16 bytes");
  DSV_REQUIRE(page_stride >= (int64_t)2 * page_size * n_kv_heads * head_dim,
              "append: page_stride smaller than one page");
  DSV_REQUIRE(aligned16(k) && aligned16(v) && aligned16(pages_layer), "append: pointers must be 16-byte aligned");
  const int row_vecs = (int)(row_bytes / 16);
  const int64_t total = (int64_t)nnz * 2 * row_vecs;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  DSV_REQUIRE(blocks < (1ll << 31), "append: too many tokens for one launch");
  const int vec_per_elem = 16 / es;
  append_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      (const uint4*)k, (const uint4*)v, k_stride_tok / vec_per_elem, v_stride_tok / vec_per_elem,
      qo_indptr, (uint4*)pages_layer, page_stride / vec_per_elem, num_pages, kv_indices, kv_indptr,
      kv_last_page_len, batch, nnz, row_vecs, page_size, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_apply_rope_inplace(void* q, void* k, int64_t q_stride_tok, int64_t k_stride_tok,
                           const int32_t* qo_indptr, const int32_t* offsets, int batch, int nnz,
                           int n_q_heads, int n_kv_heads, int head_dim, float rope_theta,
                           const float* inv_freq_host, int dtype, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "rope: unknown dtype %d", dtype);
  DSV_REQUIRE(batch >= 0 && nnz >= 0, "rope: negative batch or nnz");
  if (batch == 0 || nnz == 0) return DSV_OK;
  DSV_REQUIRE(q && k && qo_indptr && offsets, "rope: null pointer argument");
  DSV_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && head_dim <= 256, "rope: head_dim %d must be even and <= 256", head_dim);
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0, "rope: non-positive head count");
  DSV_REQUIRE(rope_theta > 0.f, "rope: rope_theta must be positive");
  DSV_REQUIRE(q_stride_tok >= (int64_t)n_q_heads * head_dim && k_stride_tok >= (int64_t)n_kv_heads * head_dim,
              "rope: token stride smaller than a row");
  RopeTable table;
  // inv_freq[i] = theta^(-2i/D): evaluated in double, rounded once to fp32
  for (int i = 0; i < head_dim / 2; ++i)
    table.inv_freq[i] = inv_freq_host != nullptr
                            ? inv_freq_host[i]
                            : (float)(1.0 / pow((double)rope_theta, (double)(2 * i) / (double)head_dim));
  const int64_t total = (int64_t)nnz * (head_dim / 2);
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  int* status = device_status_ptr();
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DSV_F32:
      rope_kernel<float><<<blocks, threads, 0, st>>>((float*)q, (float*)k, q_stride_tok, k_stride_tok, qo_indptr,
                                                     offsets, batch, nnz, n_q_heads, n_kv_heads, head_dim, table, status);
      break;
    case DSV_F16:
      rope_kernel<__half><<<blocks, threads, 0, st>>>((__half*)q, (__half*)k, q_stride_tok, k_stride_tok, qo_indptr,
                                                      offsets, batch, nnz, n_q_heads, n_kv_heads, head_dim, table, status);
      break;
    default:
      rope_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>((__nv_bfloat16*)q, (__nv_bfloat16*)k, q_stride_tok,
                                                             k_stride_tok, qo_indptr, offsets, batch, nnz, n_q_heads,
                                                             n_kv_heads, head_dim, table, status);
  }
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

}  // extern "C"
