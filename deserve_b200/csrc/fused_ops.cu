// The small kernels either side of the KV path: RMSNorm, rotary embedding fused
// into the append-scatter, and greedy (argmax) sampling. All are HBM-bound
// streaming kernels: 16-byte vectors, one pass over the data.
#include <algorithm>

#include "common.cuh"

namespace dsv {
namespace {

__device__ __forceinline__ int find_request(const int32_t* __restrict__ indptr, int batch, int tok) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(indptr + mid) <= tok) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// out[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * w, fp32 math, one rounding. One CTA per row; the
// row is kept in registers when it fits (up to kMaxVec vectors per thread), else re-read.
template <typename T, int kMaxVec>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, int64_t x_stride,
               int64_t out_stride, int dim, float eps) {
  constexpr int N = Vec16<T>::N;
  __shared__ float scratch[32];
  const int row = blockIdx.x, nvec = dim / N;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)row * x_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)row * out_stride);
  uint4 keep[kMaxVec];
  float ss = 0.f;
  int n = 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x, ++n) {
    const uint4 u = __ldg(xr + v);
    if (n < kMaxVec) keep[n] = u;
    float f[N];
    Vec16<T>::unpack(u, f);
#pragma unroll
    for (int i = 0; i < N; ++i) ss = fmaf(f[i], f[i], ss);
  }
  const float scale = rsqrtf(block_sum(ss, scratch) / (float)dim + eps);
  n = 0;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x, ++n) {
    const uint4 u = n < kMaxVec ? keep[n] : __ldg(xr + v);
    float f[N], g[N];
    Vec16<T>::unpack(u, f);
    Vec16<T>::unpack(__ldg(wr + v), g);
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = f[i] * scale * g[i];
    orow[v] = Vec16<T>::pack(f);
  }
}

// out[r, c] = silu(gu[r, c]) * gu[r, ffn + c]: the elementwise middle of the SwiGLU feed-forward on
// the output of one fused gate|up projection. Both factors are rounded to T the way the two torch
// statements round them (silu, then the product). One thread per 16-byte vector of out.
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t gu_stride, int64_t out_stride, int rows,
                int ffn) {
  constexpr int N = Vec16<T>::N;
  const int vec_per_row = ffn / N;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), v = (int)(i % vec_per_row);
    const uint4* g = reinterpret_cast<const uint4*>(gu + (int64_t)r * gu_stride) + v;
    const uint4* u = reinterpret_cast<const uint4*>(gu + (int64_t)r * gu_stride + ffn) + v;
    float a[N], b[N];
    Vec16<T>::unpack(ld_stream16(g), a);
    Vec16<T>::unpack(ld_stream16(u), b);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float s = to_f32(from_f32<T>(a[j] / (1.f + expf(-a[j]))));
      a[j] = s * b[j];
    }
    reinterpret_cast<uint4*>(out + (int64_t)r * out_stride)[v] = Vec16<T>::pack(a);
  }
}

struct RopeTable {
  float inv_freq[128];
};

// One thread per 16-byte vector of a token's q, k or v row. q is rotated in place; k is rotated
// and written straight into its page slot; v is copied into its page slot. The rotation is the
// same fp32 expression as the stand-alone rope kernel, so the bytes agree with rope + append.
template <typename T>
__global__ void __launch_bounds__(256)
rope_append_kernel(T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int64_t q_stride,
                   int64_t k_stride, int64_t v_stride, const int32_t* __restrict__ qo_indptr,
                   const int32_t* __restrict__ offsets, T* __restrict__ pages, int64_t page_stride, int64_t num_pages,
                   const int32_t* __restrict__ kv_indices, const int32_t* __restrict__ kv_indptr,
                   const int32_t* __restrict__ kv_last_page_len, int batch, int nnz, int n_q_heads, int n_kv_heads,
                   int head_dim, int page_size, RopeTable table, int* status) {
  constexpr int N = Vec16<T>::N;
  const int vph = head_dim / N;                       // vectors per head
  const int per_tok = (n_q_heads + 2 * n_kv_heads) * vph;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (int64_t)nnz * per_tok) return;
  const int tok = (int)(gid / per_tok);
  int r = (int)(gid % per_tok);
  const int req = find_request(qo_indptr, batch, tok);
  const int q0 = __ldg(qo_indptr + req), q1 = __ldg(qo_indptr + req + 1);
  const int p0 = __ldg(kv_indptr + req), p1 = __ldg(kv_indptr + req + 1);
  if (tok < q0 || tok >= q1 || p1 <= p0) {
    record_status(status, ST_BAD_REQUEST);
    return;
  }
  const int pos_in_req = tok - q0;
  const float pos = (float)(__ldg(offsets + req) + pos_in_req);
  int which;  // 0 = q, 1 = k, 2 = v
  if (r < n_q_heads * vph) which = 0;
  else if (r < (n_q_heads + n_kv_heads) * vph) { which = 1; r -= n_q_heads * vph; }
  else { which = 2; r -= (n_q_heads + n_kv_heads) * vph; }
  const int head = r / vph, vec = r % vph;
  const T* src = which == 0 ? q + (int64_t)tok * q_stride : which == 1 ? k + (int64_t)tok * k_stride : v + (int64_t)tok * v_stride;
  src += head * head_dim + vec * N;
  uint4 u = *reinterpret_cast<const uint4*>(src);
  if (which != 2) {
    float f[N];
    Vec16<T>::unpack(u, f);
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      const float angle = pos * table.inv_freq[(vec * N) / 2 + i];
      float sn, cs;
      sincosf(angle, &sn, &cs);
      const float a = f[2 * i], b = f[2 * i + 1];
      f[2 * i] = a * cs - b * sn;
      f[2 * i + 1] = a * sn + b * cs;
    }
    u = Vec16<T>::pack(f);
  }
  if (which == 0) {
    *reinterpret_cast<uint4*>(q + (int64_t)tok * q_stride + head * head_dim + vec * N) = u;
    return;
  }
  const int kv_len = (p1 - p0 - 1) * page_size + __ldg(kv_last_page_len + req);
  const int t = kv_len - (q1 - q0) + pos_in_req;
  if (t < 0) {
    record_status(status, ST_BAD_REQUEST);
    return;
  }
  const int page = __ldg(kv_indices + p0 + t / page_size);
  if (page < 0 || page >= num_pages) {
    record_status(status, ST_BAD_PAGE_ID);
    return;
  }
  T* dst = pages + (int64_t)page * page_stride +
           ((int64_t)(which - 1) * page_size + t % page_size) * n_kv_heads * head_dim + head * head_dim + vec * N;
  *reinterpret_cast<uint4*>(dst) = u;
}

// argmax of every row, lowest index among equal maxima. One CTA per row.
template <typename T>
__global__ void __launch_bounds__(256)
argmax_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab, int32_t* __restrict__ out) {
  constexpr int N = Vec16<T>::N;
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  const T* row = logits + (int64_t)blockIdx.x * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int nvec = vocab / N;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[N];
    Vec16<T>::unpack(ld_stream16(reinterpret_cast<const uint4*>(row) + v), f);
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (f[i] > best) { best = f[i]; best_i = v * N + i; }  // ascending indices: first maximum wins
  }
  for (int i = nvec * N + threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = to_f32(row[i]);
    if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) { best = s_val[w]; best_i = s_idx[w]; }
    out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_rmsnorm(const void* x, const void* weight, void* out, int64_t x_stride, int64_t out_stride, int rows, int dim,
                float eps, int dtype, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "rmsnorm: unknown dtype %d", dtype);
  DSV_REQUIRE(rows >= 0 && dim > 0, "rmsnorm: bad shape");
  if (rows == 0) return DSV_OK;
  DSV_REQUIRE(x && weight && out, "rmsnorm: null pointer argument");
  const int es = elem_size(dtype), n = 16 / es;
  DSV_REQUIRE(dim % n == 0, "rmsnorm: dim %d must be a multiple of %d", dim, n);
  DSV_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out) && (x_stride * es) % 16 == 0 && (out_stride * es) % 16 == 0,
              "rmsnorm: pointers and strides must be 16-byte aligned");
  DSV_REQUIRE(x_stride >= dim && out_stride >= dim, "rmsnorm: row stride smaller than dim");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DSV_F32:
      rmsnorm_kernel<float, 8><<<rows, 256, 0, st>>>((const float*)x, (const float*)weight, (float*)out, x_stride, out_stride, dim, eps);
      break;
    case DSV_F16:
      rmsnorm_kernel<__half, 4><<<rows, 256, 0, st>>>((const __half*)x, (const __half*)weight, (__half*)out, x_stride, out_stride, dim, eps);
      break;
    default:
      rmsnorm_kernel<__nv_bfloat16, 4><<<rows, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, x_stride, out_stride, dim, eps);
  }
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_rope_append_paged_kv(void* q, const void* k, const void* v, int64_t q_stride_tok, int64_t k_stride_tok,
                             int64_t v_stride_tok, const int32_t* qo_indptr, const int32_t* offsets, void* pages_layer,
                             int64_t page_stride, int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                             const int32_t* kv_last_page_len, int batch, int nnz, int n_q_heads, int n_kv_heads,
                             int head_dim, int page_size, float rope_theta, const float* inv_freq_host, int dtype,
                             void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "rope_append: unknown dtype %d", dtype);
  DSV_REQUIRE(batch >= 0 && nnz >= 0, "rope_append: negative batch or nnz");
  if (batch == 0 || nnz == 0) return DSV_OK;
  DSV_REQUIRE(q && k && v && qo_indptr && offsets && pages_layer && kv_indices && kv_indptr && kv_last_page_len,
              "rope_append: null pointer argument");
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && page_size > 0 && num_pages > 0, "rope_append: non-positive shape");
  const int es = elem_size(dtype), n = 16 / es;
  DSV_REQUIRE(head_dim > 0 && head_dim % n == 0 && head_dim % 2 == 0 && head_dim <= 256,
              "rope_append: head_dim %d must be even, a multiple of %d and <= 256", head_dim, n);
  DSV_REQUIRE(rope_theta > 0.f, "rope_append: rope_theta must be positive");
  DSV_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(pages_layer) && (q_stride_tok * es) % 16 == 0 &&
                  (k_stride_tok * es) % 16 == 0 && (v_stride_tok * es) % 16 == 0 && (page_stride * es) % 16 == 0,
              "rope_append: pointers and strides must be 16-byte aligned");
  DSV_REQUIRE(q_stride_tok >= (int64_t)n_q_heads * head_dim && k_stride_tok >= (int64_t)n_kv_heads * head_dim &&
                  v_stride_tok >= (int64_t)n_kv_heads * head_dim,
              "rope_append: token stride smaller than a row");
  DSV_REQUIRE(page_stride >= (int64_t)2 * page_size * n_kv_heads * head_dim, "rope_append: page_stride smaller than one page");
  RopeTable table;
  for (int i = 0; i < head_dim / 2; ++i)
    table.inv_freq[i] = inv_freq_host != nullptr
                            ? inv_freq_host[i]
                            : (float)(1.0 / pow((double)rope_theta, (double)(2 * i) / (double)head_dim));
  const int64_t total = (int64_t)nnz * (n_q_heads + 2 * n_kv_heads) * (head_dim / n);
  const int64_t blocks = (total + 255) / 256;
  DSV_REQUIRE(blocks < (1ll << 31), "rope_append: too many tokens for one launch");
  int* status = device_status_ptr();
  cudaStream_t st = (cudaStream_t)stream;
#define DSV_LAUNCH_RA(T)                                                                                             \
  rope_append_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((T*)q, (const T*)k, (const T*)v, q_stride_tok, k_stride_tok, \
                                                          v_stride_tok, qo_indptr, offsets, (T*)pages_layer,         \
                                                          page_stride, num_pages, kv_indices, kv_indptr,             \
                                                          kv_last_page_len, batch, nnz, n_q_heads, n_kv_heads,       \
                                                          head_dim, page_size, table, status)
  switch (dtype) {
    case DSV_F32: DSV_LAUNCH_RA(float); break;
    case DSV_F16: DSV_LAUNCH_RA(__half); break;
    default: DSV_LAUNCH_RA(__nv_bfloat16);
  }
#undef DSV_LAUNCH_RA
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_silu_mul(const void* gate_up, void* out, int64_t gate_up_stride, int64_t out_stride, int rows, int ffn_dim,
                 int dtype, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "silu_mul: unknown dtype %d", dtype);
  DSV_REQUIRE(rows >= 0 && ffn_dim > 0, "silu_mul: bad shape");
  if (rows == 0) return DSV_OK;
  DSV_REQUIRE(gate_up && out, "silu_mul: null pointer argument");
  const int es = elem_size(dtype), n = 16 / es;
  DSV_REQUIRE(ffn_dim % n == 0, "silu_mul: ffn_dim %d must be a multiple of %d", ffn_dim, n);
  DSV_REQUIRE(aligned16(gate_up) && aligned16(out) && (gate_up_stride * es) % 16 == 0 && (out_stride * es) % 16 == 0,
              "silu_mul: pointers and strides must be 16-byte aligned");
  DSV_REQUIRE(gate_up_stride >= 2 * (int64_t)ffn_dim && out_stride >= ffn_dim, "silu_mul: row stride smaller than a row");
  const int64_t total = (int64_t)rows * (ffn_dim / n);
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DSV_F32:
      silu_mul_kernel<float><<<grid, 256, 0, st>>>((const float*)gate_up, (float*)out, gate_up_stride, out_stride, rows, ffn_dim);
      break;
    case DSV_F16:
      silu_mul_kernel<__half><<<grid, 256, 0, st>>>((const __half*)gate_up, (__half*)out, gate_up_stride, out_stride, rows, ffn_dim);
      break;
    default:
      silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, gate_up_stride, out_stride, rows, ffn_dim);
  }
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

int dsv_greedy_sample(const void* logits, int64_t row_stride, int rows, int vocab, int32_t* tokens, int dtype,
                      void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "greedy_sample: unknown dtype %d", dtype);
  DSV_REQUIRE(rows >= 0 && vocab > 0, "greedy_sample: bad shape");
  if (rows == 0) return DSV_OK;
  DSV_REQUIRE(logits && tokens, "greedy_sample: null pointer argument");
  const int es = elem_size(dtype);
  DSV_REQUIRE(aligned16(logits) && (row_stride * es) % 16 == 0 && row_stride >= vocab,
              "greedy_sample: logits must be 16-byte aligned with a 16-byte multiple row stride");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DSV_F32: argmax_kernel<float><<<rows, 256, 0, st>>>((const float*)logits, row_stride, vocab, tokens); break;
    case DSV_F16: argmax_kernel<__half><<<rows, 256, 0, st>>>((const __half*)logits, row_stride, vocab, tokens); break;
    default: argmax_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((const __nv_bfloat16*)logits, row_stride, vocab, tokens);
  }
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

}  // extern "C"
