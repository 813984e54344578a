// Paged GQA decode attention: split-KV schedule (host), the attention kernel
// and the partial-state merge kernel.
//
// Data flow of one CTA (256 threads, 8 warps): it owns one work item =
// (request, contiguous range of that request's pages). Whole pages are staged
// from HBM into a 3-deep shared-memory ring with 16-byte cp.async copies
// (a page of one layer is one contiguous K slab followed by one contiguous V
// slab, so the copy is fully coalesced). Each warp owns one kv head; inside a
// warp the four 8-lane groups own different tokens and the 8 lanes of a group
// split head_dim, so a 128-bit shared-memory load of a group covers 128
// contiguous bytes of one token row (conflict-free). Scores are reduced over
// the 8 lanes with warp shuffles, the online softmax state (m, l, o) is kept
// per lane group in fp32 and merged by shuffles at the end of the item.
#include <algorithm>
#include <mutex>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace dsv {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr int kMaxStageBytes = 72 * 1024;
constexpr int32_t kPlanMagic = 0x44535631;  // "DSV1"
constexpr int kPlanHeader = 8;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  const void* q;
  const void* pages;
  const int32_t* kv_indices;
  const int32_t* kv_indptr;
  const int32_t* kv_last_page_len;
  void* out;
  float* lse;
  const int4* items;        // {request, first page (relative), end page (relative), partial slot or -1}
  float* part_o;            // [slots][Hq][D]
  float* part_ml;           // [slots][Hq][2]
  int64_t q_stride, out_stride, page_stride;  // elements
  int n_q_heads, n_kv_heads, page_size;
  int num_pages;            // bound of the page ids
  int hb;                   // kv heads staged per CTA (divides 8)
  int hb_log2, ps_log2;     // log2 of hb and page_size (tensor-core kernel: both are powers of two)
  int n_qblocks;            // G / QB
  float scale_log2;         // sm_scale * log2(e)
  int* status;
};

}  // namespace
}  // namespace dsv
#include "decode_mma.cuh"
#include "decode_tma.cuh"
namespace dsv {
namespace {

template <typename T, int D, int QB>
__global__ void __launch_bounds__(kThreads, 1) decode_kernel(const DecodeParams p) {
  constexpr int ES = (int)sizeof(T);
  constexpr int EPC = 16 / ES;           // elements per 16-byte vector
  constexpr int NJ = D * ES / 128;       // 128-bit loads per lane per token row
  constexpr int DL = NJ * EPC;           // head_dim elements owned by a lane (= D / 8)
  static_assert(NJ >= 1, "head_dim too small");

  extern __shared__ __align__(128) unsigned char smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane >> 3, c = lane & 7;
  const int hb = p.hb, wph = kWarps / hb;
  const int head_local = warp % hb, sub = warp / hb;
  const int ps = p.page_size;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int kv_group = blockIdx.y / p.n_qblocks, qblock = blockIdx.y % p.n_qblocks;
  const int kv_head = kv_group * hb + head_local;
  const int q_head0 = kv_head * G + qblock * QB;

  const int4 item = p.items[blockIdx.x];
  const int req = item.x;
  const int ip0 = __ldg(p.kv_indptr + req), ip1 = __ldg(p.kv_indptr + req + 1);
  const int req_pages = ip1 - ip0;
  int pb = item.y, pe = item.z;
  if (pb < 0 || pe > req_pages || pb > pe) {
    record_status(p.status, ST_BAD_PLAN);
    pb = pe = 0;
  }
  const int n_pages = pe - pb;
  const int last_len = __ldg(p.kv_last_page_len + req);
  const int32_t* idx = p.kv_indices + ip0 + pb;

  const int row_bytes = hb * D * ES;                 // one token row of the staged heads
  const int half_bytes = ps * row_bytes;             // K (or V) part of a staged page
  const int stage_bytes = 2 * half_bytes;
  const int stage_vecs = stage_bytes >> 4;
  const bool whole_page = (hb == p.n_kv_heads);
  const int row_vecs = row_bytes >> 4;
  const T* pages = reinterpret_cast<const T*>(p.pages);

  auto issue = [&](int j) {  // stage page j of the item
    int page = __ldg(idx + j);
    if (page < 0 || page >= p.num_pages) {
      record_status(p.status, ST_BAD_PAGE_ID);
      page = 0;
    }
    const unsigned char* src = reinterpret_cast<const unsigned char*>(pages + (int64_t)page * p.page_stride);
    const uint32_t dst = smem_u32(smem) + (uint32_t)((j % kStages) * stage_bytes);
    if (whole_page) {
      for (int v = tid; v < stage_vecs; v += kThreads) cp_async16(dst + (v << 4), src + ((size_t)v << 4));
    } else {
      const size_t src_row_bytes = (size_t)p.n_kv_heads * D * ES;
      const size_t head_off = (size_t)kv_group * row_bytes;
      for (int v = tid; v < stage_vecs; v += kThreads) {
        const int row = v / row_vecs, rv = v - row * row_vecs;  // row = half * ps + token
        cp_async16(dst + (v << 4), src + row * src_row_bytes + head_off + ((size_t)rv << 4));
      }
    }
  };

  // ---- q of this warp's heads, pre-scaled, in registers ---------------------
  float q[QB][DL];
  {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)req * p.q_stride;
#pragma unroll
    for (int qi = 0; qi < QB; ++qi) {
      const uint4* src = reinterpret_cast<const uint4*>(qrow + (int64_t)(q_head0 + qi) * D);
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) {
        float f[EPC];
        Vec16<T>::unpack(__ldg(src + jj * 8 + c), f);
#pragma unroll
        for (int e = 0; e < EPC; ++e) q[qi][jj * EPC + e] = f[e] * p.scale_log2;
      }
    }
  }

  float m[QB], l[QB], o[QB][DL];
#pragma unroll
  for (int qi = 0; qi < QB; ++qi) {
    m[qi] = -INFINITY;
    l[qi] = 0.f;
#pragma unroll
    for (int d = 0; d < DL; ++d) o[qi][d] = 0.f;
  }

  // ---- prologue: fill kStages-1 stages ---------------------------------------
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_pages) issue(s);
    cp_async_commit();
  }

  const int tok_step = 4 * wph;                       // tokens covered by one pass of the CTA's warps of a head
  const int n_iter = (ps + tok_step - 1) / tok_step;  // passes per page
  const int tok0 = sub * 4 + grp;                     // this lane group's first token in a page

  for (int j = 0; j < n_pages; ++j) {
    cp_async_wait<kStages - 2>();
    __syncthreads();  // page j landed for everyone; everyone is done with page j-1
    if (j + kStages - 1 < n_pages) issue(j + kStages - 1);
    cp_async_commit();

    const unsigned char* stage = smem + (j % kStages) * stage_bytes;
    const unsigned char* kbase = stage + head_local * (D * ES) + c * 16;
    const unsigned char* vbase = kbase + half_bytes;
    const int n_valid = (pb + j == req_pages - 1) ? last_len : ps;

    for (int i0 = 0; i0 < n_iter; i0 += 4) {
      float s[4][QB];
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
        for (int qi = 0; qi < QB; ++qi) s[ii][qi] = 0.f;
        const int t = tok0 + (i0 + ii) * tok_step;
        if (i0 + ii < n_iter && t < ps) {
          const unsigned char* krow = kbase + t * row_bytes;
#pragma unroll
          for (int jj = 0; jj < NJ; ++jj) {
            float f[EPC];
            Vec16<T>::unpack(*reinterpret_cast<const uint4*>(krow + jj * 128), f);
#pragma unroll
            for (int qi = 0; qi < QB; ++qi)
#pragma unroll
              for (int e = 0; e < EPC; ++e) s[ii][qi] = fmaf(q[qi][jj * EPC + e], f[e], s[ii][qi]);
          }
        }
      }
      // reduce every score over the 8 lanes that split head_dim
#pragma unroll
      for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int qi = 0; qi < QB; ++qi) {
          float x = s[ii][qi];
          x += __shfl_xor_sync(0xffffffffu, x, 1);
          x += __shfl_xor_sync(0xffffffffu, x, 2);
          x += __shfl_xor_sync(0xffffffffu, x, 4);
          s[ii][qi] = x;
        }
      bool valid[4];
      bool any = false;
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        const int t = tok0 + (i0 + ii) * tok_step;
        valid[ii] = (i0 + ii < n_iter) && (t < n_valid);
        any |= valid[ii];
      }
      if (any) {  // uniform inside an 8-lane group; no shuffles below
#pragma unroll
        for (int qi = 0; qi < QB; ++qi) {
          float mx = m[qi];
#pragma unroll
          for (int ii = 0; ii < 4; ++ii)
            if (valid[ii]) mx = fmaxf(mx, s[ii][qi]);
          const float sc = exp2f(m[qi] - mx);  // m = -inf on first use -> 0
          m[qi] = mx;
          float lsum = l[qi] * sc;
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            const float pv = valid[ii] ? exp2f(s[ii][qi] - mx) : 0.f;
            s[ii][qi] = pv;
            lsum += pv;
          }
          l[qi] = lsum;
#pragma unroll
          for (int d = 0; d < DL; ++d) o[qi][d] *= sc;
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          if (valid[ii]) {
            const int t = tok0 + (i0 + ii) * tok_step;
            const unsigned char* vrow = vbase + t * row_bytes;
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
              float f[EPC];
              Vec16<T>::unpack(*reinterpret_cast<const uint4*>(vrow + jj * 128), f);
#pragma unroll
              for (int qi = 0; qi < QB; ++qi)
#pragma unroll
                for (int e = 0; e < EPC; ++e) o[qi][jj * EPC + e] = fmaf(s[ii][qi], f[e], o[qi][jj * EPC + e]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- merge the four lane groups of the warp --------------------------------
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
    for (int qi = 0; qi < QB; ++qi) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[qi], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[qi], off);
      const float mx = fmaxf(m[qi], m2);
      const float a1 = (m[qi] == -INFINITY) ? 0.f : exp2f(m[qi] - mx);
      const float a2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mx);
      m[qi] = mx;
      l[qi] = l[qi] * a1 + l2 * a2;
#pragma unroll
      for (int d = 0; d < DL; ++d) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[qi][d], off);
        o[qi][d] = o[qi][d] * a1 + o2 * a2;
      }
    }
  }

  // ---- merge the warps that share a head, through shared memory ---------------
  __syncthreads();  // ring no longer read
  float* sc_o = reinterpret_cast<float*>(smem);                 // [warp][QB][D]
  float* sc_ml = sc_o + kWarps * QB * D;                         // [warp][QB][2]
  if (grp == 0) {
#pragma unroll
    for (int qi = 0; qi < QB; ++qi) {
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj)
#pragma unroll
        for (int e = 0; e < EPC; ++e)
          sc_o[(warp * QB + qi) * D + (jj * 8 + c) * EPC + e] = o[qi][jj * EPC + e];
      if (c == 0) {
        sc_ml[(warp * QB + qi) * 2 + 0] = m[qi];
        sc_ml[(warp * QB + qi) * 2 + 1] = l[qi];
      }
    }
  }
  __syncthreads();

  const int slot = item.w;
  for (int x = tid; x < hb * QB * D; x += kThreads) {
    const int d = x % D, qi = (x / D) % QB, hl = x / (D * QB);
    float mx = -INFINITY;
    for (int s2 = 0; s2 < wph; ++s2) mx = fmaxf(mx, sc_ml[((s2 * hb + hl) * QB + qi) * 2]);
    float lsum = 0.f, acc = 0.f;
    for (int s2 = 0; s2 < wph; ++s2) {
      const int w2 = s2 * hb + hl;
      const float mw = sc_ml[(w2 * QB + qi) * 2];
      const float a = (mw == -INFINITY) ? 0.f : exp2f(mw - mx);
      lsum += sc_ml[(w2 * QB + qi) * 2 + 1] * a;
      acc += sc_o[(w2 * QB + qi) * D + d] * a;
    }
    const int qh = (kv_group * hb + hl) * G + qblock * QB + qi;
    if (slot < 0) {
      const float r = lsum > 0.f ? acc / lsum : 0.f;
      reinterpret_cast<T*>(p.out)[(int64_t)req * p.out_stride + (int64_t)qh * D + d] = from_f32<T>(r);
      if (p.lse != nullptr && d == 0)
        p.lse[(int64_t)req * p.n_q_heads + qh] = lsum > 0.f ? (mx + log2f(lsum)) * kLn2 : -INFINITY;
    } else {
      p.part_o[((int64_t)slot * p.n_q_heads + qh) * D + d] = acc;
      if (d == 0) {
        p.part_ml[((int64_t)slot * p.n_q_heads + qh) * 2 + 0] = mx;
        p.part_ml[((int64_t)slot * p.n_q_heads + qh) * 2 + 1] = lsum;
      }
    }
  }
}

// One CTA of 128 threads per (request, q head): fold that request's partial states.
// The weights 2^(m_s - max m) are computed once, cooperatively, into shared memory; then thread d
// sums its head_dim element over all parts with independent (pipelined) loads. A request cut into
// hundreds of parts (one long sequence spread over the whole machine) costs a few microseconds.
constexpr int kMergeThreads = 128;
constexpr int kMergeChunk = 512;  // parts handled per pass (shared-memory weights)

template <typename T>
__global__ void __launch_bounds__(kMergeThreads)
merge_kernel(const int2* __restrict__ merge, const float* __restrict__ part_o,
             const float* __restrict__ part_ml, T* __restrict__ out, float* __restrict__ lse,
             int64_t out_stride, int n_q_heads, int head_dim) {
  __shared__ float w[kMergeChunk];
  __shared__ float red[kMergeThreads / 32];
  __shared__ float bcast[2];
  const int req = blockIdx.x, qh = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int2 mi = merge[req];
  if (mi.y <= 1) return;  // written directly by the attention kernel
  const float* ml = part_ml + ((int64_t)mi.x * n_q_heads + qh) * 2;
  const int64_t ml_step = (int64_t)n_q_heads * 2;
  // maximum of the parts' running maxima
  float mx = -INFINITY;
  for (int s = tid; s < mi.y; s += kMergeThreads) mx = fmaxf(mx, ml[s * ml_step]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = red[0];
    for (int i = 1; i < kMergeThreads / 32; ++i) t = fmaxf(t, red[i]);
    bcast[0] = t;
  }
  __syncthreads();
  mx = bcast[0];
  float acc[2] = {0.f, 0.f};  // head_dim <= 256: up to two elements per thread
  float lsum = 0.f;
  for (int s0 = 0; s0 < mi.y; s0 += kMergeChunk) {
    const int n = min(kMergeChunk, mi.y - s0);
    __syncthreads();  // w from the previous pass is no longer read
    for (int s = tid; s < n; s += kMergeThreads) {
      const float ms = ml[(s0 + s) * ml_step];
      const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
      w[s] = a;
      lsum += ml[(s0 + s) * ml_step + 1] * a;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int d = tid + k * kMergeThreads;
      if (d < head_dim) {
        const float* po = part_o + ((int64_t)(mi.x + s0) * n_q_heads + qh) * head_dim + d;
        const int64_t step = (int64_t)n_q_heads * head_dim;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int s = 0;
        for (; s + 4 <= n; s += 4) {
          a0 = fmaf(po[(s + 0) * step], w[s + 0], a0);
          a1 = fmaf(po[(s + 1) * step], w[s + 1], a1);
          a2 = fmaf(po[(s + 2) * step], w[s + 2], a2);
          a3 = fmaf(po[(s + 3) * step], w[s + 3], a3);
        }
        for (; s < n; ++s) a0 = fmaf(po[s * step], w[s], a0);
        acc[k] += (a0 + a1) + (a2 + a3);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  __syncthreads();
  if (lane == 0) red[warp] = lsum;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < kMergeThreads / 32; ++i) t += red[i];
    bcast[1] = t;
  }
  __syncthreads();
  lsum = bcast[1];
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int d = tid + k * kMergeThreads;
    if (d < head_dim) out[(int64_t)req * out_stride + (int64_t)qh * head_dim + d] = from_f32<T>(acc[k] * inv);
  }
  if (lse != nullptr && tid == 0)
    lse[(int64_t)req * n_q_heads + qh] = lsum > 0.f ? (mx + log2f(lsum)) * kLn2 : -INFINITY;
}

// kv heads staged per CTA: the largest divisor of 8 that divides n_kv_heads and
// keeps one staged page within the per-stage shared-memory budget.
int pick_hb(int n_kv_heads, int head_dim, int page_size, int es) {
  for (int hb = 8; hb >= 1; hb >>= 1) {
    if (n_kv_heads % hb != 0) continue;
    if ((int64_t)2 * page_size * hb * head_dim * es <= kMaxStageBytes) return hb;
  }
  return 0;
}

int pick_qb(int group) {
  if (group % 4 == 0) return 4;
  if (group % 2 == 0) return 2;
  return 1;
}

template <typename T, int D>
cudaError_t launch_decode(const DecodeParams& p, int qb, dim3 grid, size_t smem, cudaStream_t st) {
  auto go = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, kThreads, smem, st>>>(p);
    return cudaGetLastError();
  };
  switch (qb) {
    case 4: return go(decode_kernel<T, D, 4>);
    case 2: return go(decode_kernel<T, D, 2>);
    default: return go(decode_kernel<T, D, 1>);
  }
}

template <typename T, int D>
cudaError_t launch_decode_mma(const DecodeParams& p, bool hi, dim3 grid, size_t smem, cudaStream_t st) {
  auto go = [&](auto kernel) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kernel<<<grid, mma_decode::kThreads, smem, st>>>(p);
    return cudaGetLastError();
  };
  return hi ? go(mma_decode::decode_mma_kernel<T, D, true>) : go(mma_decode::decode_mma_kernel<T, D, false>);
}

inline int ilog2_exact(int x) {  // log2 of a power of two, -1 otherwise
  if (x <= 0 || (x & (x - 1)) != 0) return -1;
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

template <typename T>
cudaError_t launch_decode_d(const DecodeParams& p, int head_dim, int qb, dim3 grid, size_t smem, cudaStream_t st) {
  if (head_dim == 128) return launch_decode<T, 128>(p, qb, grid, smem, st);
  return launch_decode<T, 64>(p, qb, grid, smem, st);
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_decode_plan(const int32_t* kv_indptr_host, int batch, int n_q_heads, int n_kv_heads,
                    int head_dim, int page_size, int dtype, int sm_count, int32_t* plan_host,
                    int64_t plan_capacity_i32, int64_t* plan_used_i32, int64_t* workspace_bytes) {
  using namespace dsv;
  DSV_REQUIRE(kv_indptr_host && plan_host && plan_used_i32 && workspace_bytes, "decode_plan: null pointer argument");
  DSV_REQUIRE(batch >= 0, "decode_plan: negative batch");
  DSV_REQUIRE(dtype_ok(dtype), "decode_plan: unknown dtype %d", dtype);
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
              "decode_plan: n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, n_kv_heads);
  DSV_REQUIRE(head_dim == 64 || head_dim == 128, "decode_plan: head_dim %d not in {64,128}", head_dim);
  DSV_REQUIRE(page_size > 0, "decode_plan: page_size must be positive");
  if (sm_count <= 0) sm_count = 148;
  int64_t total_pages = 0;
  int max_pages = 0;
  for (int i = 0; i < batch; ++i) {
    const int n = kv_indptr_host[i + 1] - kv_indptr_host[i];
    DSV_REQUIRE(n >= 0, "decode_plan: kv_indptr not monotone at %d", i);
    total_pages += n;
    max_pages = std::max(max_pages, n);
  }
  // Chunk length (pages): the smallest c for which the item count fits the
  // target of ~4 items per SM, but never shorter than ~256 tokens so that the
  // pipeline fill of an item stays amortised.
  const int64_t target_items = std::max<int64_t>((int64_t)4 * sm_count, batch);
  const int min_chunk = std::max(1, 256 / page_size);
  auto count_items = [&](int c) {
    int64_t n = 0;
    for (int i = 0; i < batch; ++i) {
      const int np = kv_indptr_host[i + 1] - kv_indptr_host[i];
      n += std::max(1, (np + c - 1) / c);
    }
    return n;
  };
  int lo = min_chunk, hi = std::max(min_chunk, max_pages);
  while (lo < hi) {
    const int mid = lo + (hi - lo) / 2;
    if (count_items(mid) <= target_items) hi = mid; else lo = mid + 1;
  }
  int chunk = lo;
  // Small batches (a 128-sequence microbatch with contexts of a few hundred tokens streams
  // ~0.3 GB per launch): the rule above cuts every request into several short items, and then the
  // fixed cost of an item (tensor-map fetch, q load, ring fill and drain, partial-state write) and
  // the extra merge launch weigh as much as the streaming itself. For such launches a few longer
  // chunk lengths are compared on a model of the launch: items handed longest first to sm_count
  // CTAs, an item costing its pages plus a fixed overhead, a merge costing a fixed amount when any
  // request is split. The rule's choice stays unless a candidate is predicted to be clearly faster.
  if (total_pages <= (int64_t)96 * sm_count && batch > 0) {
    const int64_t page_bytes = (int64_t)2 * page_size * n_kv_heads * head_dim * elem_size(dtype);
    const double ovh = std::max<double>(1.0, (512.0 * 1024.0) / (double)page_bytes);  // ~0.5 MB of streaming time
    const double merge_cost = 1.5 * ovh;
    std::vector<int> lens;
    auto predicted = [&](int c) {
      lens.clear();
      bool split = false;
      for (int i = 0; i < batch; ++i) {
        const int np = kv_indptr_host[i + 1] - kv_indptr_host[i];
        const int parts = std::max(1, (np + c - 1) / c);
        split = split || parts > 1;
        const int base = np / parts, extra = np % parts;
        for (int p = 0; p < parts; ++p) lens.push_back(base + (p < extra ? 1 : 0));
      }
      std::sort(lens.begin(), lens.end(), std::greater<int>());
      double makespan = 0.0;
      if ((int)lens.size() <= sm_count) {
        makespan = lens.empty() ? 0.0 : lens[0] + ovh;
      } else {
        std::vector<double> busy(sm_count);  // min-heap of the times at which a CTA slot becomes free
        for (int k = 0; k < sm_count; ++k) busy[k] = lens[k] + ovh;
        std::make_heap(busy.begin(), busy.end(), std::greater<double>());
        for (size_t k = sm_count; k < lens.size(); ++k) {
          std::pop_heap(busy.begin(), busy.end(), std::greater<double>());
          busy.back() += lens[k] + ovh;
          std::push_heap(busy.begin(), busy.end(), std::greater<double>());
        }
        for (double t : busy) makespan = std::max(makespan, t);
      }
      return makespan + (split ? merge_cost : 0.0);
    };
    const double base_cost = predicted(chunk);
    double best_cost = base_cost;
    int best = chunk;
    // candidates: the longest request in 1..4 parts, and chunk lengths that make the item count about
    // 1, 2 or 3 per CTA (each a little longer too: the per-request rounding adds items)
    int cand[4 + 9];
    int n_cand = 0;
    for (int parts = 1; parts <= 4; ++parts) cand[n_cand++] = (max_pages + parts - 1) / parts;
    for (int per_cta = 1; per_cta <= 3; ++per_cta) {
      const int c = (int)((total_pages + (int64_t)per_cta * sm_count - 1) / ((int64_t)per_cta * sm_count));
      cand[n_cand++] = c;
      cand[n_cand++] = c + std::max(1, c / 8);
      cand[n_cand++] = c + std::max(2, c / 4);
    }
    for (int k = 0; k < n_cand; ++k) {
      const int c = std::max(min_chunk, cand[k]);
      if (c <= chunk || c > std::max(min_chunk, max_pages) || count_items(c) > target_items) continue;
      const double cost = predicted(c);
      if (cost < best_cost) { best_cost = cost; best = c; }
    }
    if (best_cost < 0.93 * base_cost) chunk = best;
  }
  const int64_t n_items = count_items(chunk);
  const int64_t need = kPlanHeader + 4 * n_items + 2 * (int64_t)batch;
  *plan_used_i32 = need;
  if (need > plan_capacity_i32)
    return fail(DSV_E_WORKSPACE, "decode_plan: plan needs %lld int32, capacity %lld", (long long)need,
                (long long)plan_capacity_i32);

  struct Item { int req, pb, pe, slot; };
  std::vector<Item> items;
  items.reserve((size_t)n_items);
  int32_t* merge = plan_host + kPlanHeader + 4 * n_items;
  int slots = 0;
  for (int i = 0; i < batch; ++i) {
    const int np = kv_indptr_host[i + 1] - kv_indptr_host[i];
    const int parts = std::max(1, (np + chunk - 1) / chunk);
    merge[2 * i] = parts > 1 ? slots : -1;
    merge[2 * i + 1] = parts;
    // equal-sized parts rather than full chunks plus a stub
    const int base = np / parts, extra = np % parts;
    int at = 0;
    for (int s = 0; s < parts; ++s) {
      const int len = base + (s < extra ? 1 : 0);
      items.push_back({i, at, at + len, parts > 1 ? slots + s : -1});
      at += len;
    }
    if (parts > 1) slots += parts;
  }
  // longest first: the hardware scheduler hands items to SMs in order
  std::stable_sort(items.begin(), items.end(),
                   [](const Item& a, const Item& b) { return (a.pe - a.pb) > (b.pe - b.pb); });
  plan_host[0] = kPlanMagic;
  plan_host[1] = (int32_t)n_items;
  plan_host[2] = slots;
  plan_host[3] = chunk;
  plan_host[4] = batch;
  plan_host[5] = kPlanHeader;
  plan_host[6] = (int32_t)(kPlanHeader + 4 * n_items);
  plan_host[7] = n_q_heads;
  for (int64_t k = 0; k < n_items; ++k) {
    int32_t* it = plan_host + kPlanHeader + 4 * k;
    it[0] = items[k].req; it[1] = items[k].pb; it[2] = items[k].pe; it[3] = items[k].slot;
  }
  *workspace_bytes = (int64_t)slots * n_q_heads * (head_dim + 2) * (int64_t)sizeof(float);
  return DSV_OK;
}

int dsv_paged_decode(const void* q, int64_t q_stride_tok, const void* pages_layer,
                     int64_t page_stride, int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                     const int32_t* kv_last_page_len, void* out, int64_t out_stride_tok,
                     float* lse, const int32_t* plan_host, const int32_t* plan_dev,
                     void* workspace, int64_t workspace_bytes, int batch, int n_q_heads,
                     int n_kv_heads, int head_dim, int page_size, int dtype, float sm_scale,
                     void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "decode: unknown dtype %d", dtype);
  DSV_REQUIRE(batch >= 0, "decode: negative batch");
  if (batch == 0) return DSV_OK;
  DSV_REQUIRE(q && pages_layer && kv_indices && kv_indptr && kv_last_page_len && out && plan_host && plan_dev,
              "decode: null pointer argument");
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0,
              "decode: n_q_heads (%d) must be a positive multiple of n_kv_heads (%d)", n_q_heads, n_kv_heads);
  DSV_REQUIRE(head_dim == 64 || head_dim == 128, "decode: head_dim %d not in {64,128}", head_dim);
  DSV_REQUIRE(page_size > 0, "decode: page_size must be positive");
  DSV_REQUIRE(num_pages > 0 && num_pages < (1ll << 30), "decode: num_pages (%lld) out of range", (long long)num_pages);
  DSV_REQUIRE(plan_host[0] == kPlanMagic && plan_host[4] == batch && plan_host[7] == n_q_heads,
              "decode: plan does not belong to this batch (magic %x, batch %d, heads %d)", plan_host[0],
              plan_host[4], plan_host[7]);
  const int es = elem_size(dtype);
  DSV_REQUIRE(aligned16(q) && aligned16(pages_layer) && aligned16(out), "decode: pointers must be 16-byte aligned");
  DSV_REQUIRE((q_stride_tok * es) % 16 == 0 && (page_stride * es) % 16 == 0, "decode: strides must be multiples of 16 bytes");
  DSV_REQUIRE(q_stride_tok >= (int64_t)n_q_heads * head_dim && out_stride_tok >= (int64_t)n_q_heads * head_dim,
              "decode: token stride smaller than a row");
  DSV_REQUIRE(page_stride >= (int64_t)2 * page_size * n_kv_heads * head_dim, "decode: page_stride smaller than one page");
  const int hb = pick_hb(n_kv_heads, head_dim, page_size, es);
  if (hb == 0)
    return fail(DSV_E_UNSUPPORTED, "decode: no staging shape for n_kv_heads=%d head_dim=%d page_size=%d", n_kv_heads,
                head_dim, page_size);
  const int G = n_q_heads / n_kv_heads;
  const int qb = pick_qb(G);
  const int n_items = plan_host[1], slots = plan_host[2];
  const int64_t ws_need = (int64_t)slots * n_q_heads * (head_dim + 2) * (int64_t)sizeof(float);
  if (ws_need > 0 && (workspace == nullptr || workspace_bytes < ws_need))
    return fail(DSV_E_WORKSPACE, "decode: workspace needs %lld bytes, got %lld", (long long)ws_need,
                (long long)workspace_bytes);
  DSV_REQUIRE(ws_need == 0 || aligned16(workspace), "decode: workspace must be 16-byte aligned");

  DecodeParams p;
  p.q = q; p.pages = pages_layer; p.kv_indices = kv_indices; p.kv_indptr = kv_indptr;
  p.kv_last_page_len = kv_last_page_len; p.out = out; p.lse = lse;
  p.items = reinterpret_cast<const int4*>(plan_dev + plan_host[5]);
  DSV_REQUIRE(aligned16(p.items), "decode: device plan must be 16-byte aligned");
  p.part_o = static_cast<float*>(workspace);
  p.part_ml = p.part_o + (int64_t)slots * n_q_heads * head_dim;
  p.q_stride = q_stride_tok; p.out_stride = out_stride_tok; p.page_stride = page_stride;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.num_pages = (int)num_pages;
  p.hb = hb; p.hb_log2 = 0; p.ps_log2 = 0; p.n_qblocks = G / qb; p.scale_log2 = sm_scale * kLog2e; p.status = device_status_ptr();

  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  // 16-bit K/V with a GQA group of at most 16 heads and power-of-two page size:
  // tensor-core kernel. Everything else (fp32 above all): CUDA-core kernel.
  int hb2 = 8;
  while (hb2 > 1 && n_kv_heads % hb2 != 0) hb2 >>= 1;
  const int ps_log2 = ilog2_exact(page_size);
  if (dtype != DSV_F32 && G <= 16 && ps_log2 >= 0) {
    p.hb = hb2; p.hb_log2 = ilog2_exact(hb2); p.ps_log2 = ps_log2;
    const bool hi = G > 8;
    const size_t stage = (size_t)512 * head_dim;  // 2 halves x 128 rows x head_dim x 2 bytes
    const size_t scratch = (size_t)mma_decode::kWarps * (hi ? 16 : 8) * (head_dim + 2) * sizeof(float);
    const size_t smem = std::max(stage * mma_decode::kStages, scratch);
    const dim3 grid((unsigned)n_items, (unsigned)(n_kv_heads / hb2));
    CUtensorMap tmap;
    const bool use_tma = ps_log2 >= 3 && page_stride == (int64_t)2 * page_size * n_kv_heads * head_dim &&
                         tma_decode::make_pages_tensor_map(&tmap, pages_layer, page_stride, num_pages, page_size,
                                                           n_kv_heads, head_dim, hb2, dtype == DSV_BF16);
    if (use_tma) {
      const size_t tsmem = std::max(stage * tma_decode::kStages + 1024 + 64, scratch + 1024);
      auto go = [&](auto kernel) -> cudaError_t {
        cudaError_t er = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem);
        if (er != cudaSuccess) return er;
        kernel<<<grid, tma_decode::kThreads, tsmem, st>>>(tmap, p);
        return cudaGetLastError();
      };
      if (dtype == DSV_F16)
        e = head_dim == 128 ? (hi ? go(tma_decode::decode_tma_kernel<__half, 128, true>)
                                  : go(tma_decode::decode_tma_kernel<__half, 128, false>))
                            : (hi ? go(tma_decode::decode_tma_kernel<__half, 64, true>)
                                  : go(tma_decode::decode_tma_kernel<__half, 64, false>));
      else
        e = head_dim == 128 ? (hi ? go(tma_decode::decode_tma_kernel<__nv_bfloat16, 128, true>)
                                  : go(tma_decode::decode_tma_kernel<__nv_bfloat16, 128, false>))
                            : (hi ? go(tma_decode::decode_tma_kernel<__nv_bfloat16, 64, true>)
                                  : go(tma_decode::decode_tma_kernel<__nv_bfloat16, 64, false>));
    } else if (dtype == DSV_F16)
      e = head_dim == 128 ? launch_decode_mma<__half, 128>(p, hi, grid, smem, st)
                          : launch_decode_mma<__half, 64>(p, hi, grid, smem, st);
    else
      e = head_dim == 128 ? launch_decode_mma<__nv_bfloat16, 128>(p, hi, grid, smem, st)
                          : launch_decode_mma<__nv_bfloat16, 64>(p, hi, grid, smem, st);
  } else {
    const size_t stage_bytes = (size_t)2 * page_size * hb * head_dim * es;
    const size_t scratch = (size_t)kWarps * qb * (head_dim + 2) * sizeof(float);
    const size_t smem = std::max(stage_bytes * kStages, scratch);
    const dim3 grid((unsigned)n_items, (unsigned)((n_kv_heads / hb) * (G / qb)));
    switch (dtype) {
      case DSV_F32: e = launch_decode_d<float>(p, head_dim, qb, grid, smem, st); break;
      case DSV_F16: e = launch_decode_d<__half>(p, head_dim, qb, grid, smem, st); break;
      default: e = launch_decode_d<__nv_bfloat16>(p, head_dim, qb, grid, smem, st);
    }
  }
  if (e != cudaSuccess) return fail(DSV_E_CUDA, "decode launch failed: %s", cudaGetErrorString(e));

  if (slots > 0) {
    const int2* merge = reinterpret_cast<const int2*>(plan_dev + plan_host[6]);
    const dim3 mgrid((unsigned)batch, (unsigned)n_q_heads);
    switch (dtype) {
      case DSV_F32:
        merge_kernel<float><<<mgrid, kMergeThreads, 0, st>>>(merge, p.part_o, p.part_ml, (float*)out, lse, out_stride_tok, n_q_heads, head_dim);
        break;
      case DSV_F16:
        merge_kernel<__half><<<mgrid, kMergeThreads, 0, st>>>(merge, p.part_o, p.part_ml, (__half*)out, lse, out_stride_tok, n_q_heads, head_dim);
        break;
      default:
        merge_kernel<__nv_bfloat16><<<mgrid, kMergeThreads, 0, st>>>(merge, p.part_o, p.part_ml, (__nv_bfloat16*)out, lse, out_stride_tok, n_q_heads, head_dim);
    }
    DSV_CUDA(cudaGetLastError());
  }
  return DSV_OK;
}

// ---- decode without a caller workspace ------------------------------------------------------
// Scratch for the split-KV partial states of dsv_paged_decode_static. In host code this
// name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_decode_scratch[DSV_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxScratchDevices = 64;
void* g_scratch_ptr[kMaxScratchDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of g_decode_scratch on the current device, resolved once per device
// (under a lock: two host threads may make their first call on a device at the same time).
int static_scratch(void** out) {
  int dev = -1;
  DSV_CUDA(cudaGetDevice(&dev));
  DSV_REQUIRE(dev >= 0 && dev < kMaxScratchDevices, "decode_static: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    DSV_CUDA(cudaGetSymbolAddress(&ptr, g_decode_scratch));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return DSV_OK;
}
}  // namespace

int dsv_paged_decode_static(const void* q, int64_t q_stride_tok, const void* pages_layer,
                            int64_t page_stride, int64_t num_pages, const int32_t* kv_indices,
                            const int32_t* kv_indptr, const int32_t* kv_last_page_len, void* out,
                            int64_t out_stride_tok, float* lse, const int32_t* plan_host,
                            const int32_t* plan_dev, int batch, int n_q_heads, int n_kv_heads,
                            int head_dim, int page_size, int dtype, float sm_scale, void* stream) {
  using namespace dsv;
  if (batch == 0) return DSV_OK;
  DSV_REQUIRE(plan_host != nullptr, "decode_static: null plan");
  DSV_REQUIRE(plan_host[0] == kPlanMagic && plan_host[2] >= 0 && n_q_heads > 0 && head_dim > 0,
              "decode_static: not a decode plan");
  const int64_t need = (int64_t)plan_host[2] * n_q_heads * (head_dim + 2) * (int64_t)sizeof(float);
  if (need > (int64_t)DSV_STATIC_SCRATCH_BYTES)
    return fail(DSV_E_WORKSPACE,
                "decode_static: this plan's partial states need %lld bytes, the built-in scratch holds %lld; "
                "use dsv_paged_decode with a caller workspace",
                (long long)need, (long long)DSV_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != DSV_OK) return rc;
  return dsv_paged_decode(q, q_stride_tok, pages_layer, page_stride, num_pages, kv_indices, kv_indptr,
                          kv_last_page_len, out, out_stride_tok, lse, plan_host, plan_dev, scratch,
                          (int64_t)DSV_STATIC_SCRATCH_BYTES, batch, n_q_heads, n_kv_heads, head_dim, page_size,
                          dtype, sm_scale, stream);
}

// ---- self-test of the bounded-wait machinery ---------------------------------------------------
namespace {
// One thread waits on an mbarrier phase that nobody will ever complete, with a small poll limit;
// the wait must give up, record ST_WAIT_TIMEOUT and let the kernel end normally.
__global__ void wait_timeout_selftest_kernel(int polls, int* status) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t addr = dsv::smem_u32(&bar);
  dsv::tma_decode::mbar_init(addr, 1);
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  bool done = false;
  for (int i = 0; i < polls && !done; ++i) done = dsv::tma_decode::mbar_try_wait(addr, 0);
  if (!done) dsv::record_status(status, dsv::ST_WAIT_TIMEOUT);
}
}  // namespace

int dsv_selftest_wait_timeout(int polls, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(polls > 0 && polls <= (1 << 20), "selftest: polls must be in [1, 2^20]");
  wait_timeout_selftest_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(polls, device_status_ptr());
  DSV_CUDA(cudaGetLastError());
  return DSV_OK;
}

}  // extern "C"
