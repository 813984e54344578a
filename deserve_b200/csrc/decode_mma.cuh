// Paged GQA decode attention for 16-bit K/V: the q.K^T and P.V products of a
// GQA group are small dense contractions (G x 16 tokens x head_dim), issued as
// warp-level mma.sync.m16n8k16 with the group's q heads padded into the 16 rows
// of the A operand; the online softmax runs on the accumulator fragments with
// quad shuffles. Included by decode.cu (shares DecodeParams and the plan).
//
// CTA = 8 warps. A tile is 16*WPH tokens x HB kv heads (HB*WPH = 8), K then V,
// 512*head_dim bytes, staged through a 3-deep shared-memory ring with 16-byte
// cp.async copies. Rows of a (head, token) are head_dim*2 bytes; the 16-byte
// chunk c of token t is stored at chunk c ^ (t & 7), so the 8 row addresses of
// every ldmatrix fall in 8 different bank groups.
#pragma once

#include "common.cuh"

namespace dsv {
namespace mma_decode {

constexpr int kWarps = 8;
constexpr int kThreads = 256;
constexpr int kStages = 3;

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 16-byte cp.async that writes zeros when `valid` is false (src-size 0).
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gptr), "r"(n) : "memory");
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// HI: the GQA group has more than 8 q heads, so rows 8..15 of the fragments are live.
template <typename T, int D, bool HI>
__global__ void __launch_bounds__(kThreads, 1) decode_mma_kernel(const DecodeParams p) {
  constexpr int ROWB = D * 2;        // bytes of one (head, token) row
  constexpr int CPR = D / 8;         // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;
  constexpr int HALF = 128 * ROWB;   // K (or V) part of a stage: HB*TTOK = 128 rows
  constexpr int STAGE = 2 * HALF;
  constexpr int ITERS = 2 * 128 * CPR / kThreads;

  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tg = lane & 3;
  const int hb_log = p.hb_log2, hb = 1 << hb_log;
  const int wph = kWarps >> hb_log, ttok = 16 * wph;
  const int head_local = warp & (hb - 1), sub = warp >> hb_log;
  const int ps_log = p.ps_log2, ps = 1 << ps_log;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int kv_group = blockIdx.y;
  const int kv_head = kv_group * hb + head_local;

  const int4 item = p.items[blockIdx.x];
  const int req = item.x;
  const int ip0 = __ldg(p.kv_indptr + req), ip1 = __ldg(p.kv_indptr + req + 1);
  const int req_pages = ip1 - ip0;
  int pb = item.y, pe = item.z;
  if (pb < 0 || pe > req_pages || pb > pe) {
    record_status(p.status, ST_BAD_PLAN);
    pb = pe = 0;
  }
  const int kv_len = req_pages > 0 ? (req_pages - 1) * ps + __ldg(p.kv_last_page_len + req) : 0;
  const int tok_begin = pb << ps_log;
  const int tok_end = min(pe << ps_log, kv_len);
  const int n_tok = max(tok_end - tok_begin, 0);
  const int n_tiles = (n_tok + ttok - 1) / ttok;
  const int32_t* idx = p.kv_indices + ip0;
  const unsigned char* pages = reinterpret_cast<const unsigned char*>(p.pages);
  const int64_t page_stride_b = p.page_stride * 2;
  const int src_row_b = p.n_kv_heads * ROWB;          // bytes of one token row in a page (all heads)
  const int src_half_b = ps * src_row_b;              // K part of a page

  // ---- staging: thread -> (chunk, head) fixed, rows advance with the trip ----------
  auto issue = [&](int tile) {
    const uint32_t dst_stage = smem_base + (uint32_t)((tile % kStages) * STAGE);
    const int t0 = tok_begin + tile * ttok;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int ci = tid + it * kThreads;
      const int c = ci & (CPR - 1);
      const int row = ci / CPR;                 // 0..255: half * 128 + token * hb + head
      const int half = row >> 7, rr = row & 127;
      const int t = rr >> hb_log, h = rr & (hb - 1);
      const int gt = t0 + t;
      const bool valid = gt < tok_end;
      int page = 0;
      if (valid) {
        page = __ldg(idx + (gt >> ps_log));
        if (page < 0 || page >= p.num_pages) {
          record_status(p.status, ST_BAD_PAGE_ID);
          page = 0;
        }
      }
      const unsigned char* src = pages + (int64_t)page * page_stride_b + (size_t)half * src_half_b +
                                 (size_t)(gt & (ps - 1)) * src_row_b + (size_t)(kv_group * hb + h) * ROWB + c * 16;
      const uint32_t dst = dst_stage + half * HALF + (h * ttok + t) * ROWB + ((c ^ (t & 7)) << 4);
      cp_async16_zfill(dst, src, valid);
    }
  };

  // ---- q fragments of this warp's kv head (rows = q heads of the group) ----------------
  uint32_t qa[KSTEPS][4];
  {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)req * p.q_stride + (int64_t)kv_head * G * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + tg * 2;
      qa[kk][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + g * D + d0) : 0u;
      qa[kk][2] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + g * D + d0 + 8) : 0u;
      qa[kk][1] = (HI && g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * D + d0) : 0u;
      qa[kk][3] = (HI && g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * D + d0 + 8) : 0u;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g+8 (scaled log2 domain)
  const float sc = p.scale_log2;

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) issue(s);
    cp_async_commit();
  }

  // lane-dependent parts of the ldmatrix row addresses
  const int lr = lane & 7, lm = lane >> 3;
  const int k_tl = lr + ((lm >> 1) << 3), k_cx = lm & 1;   // K: matrices (tok lo, c), (tok lo, c+1), (tok hi, c), (tok hi, c+1)
  const int v_tl = lr + ((lm & 1) << 3), v_cx = lm >> 1;   // V: matrices (tok lo, c), (tok hi, c), (tok lo, c+1), (tok hi, c+1)
  const uint32_t warp_rows = (uint32_t)((head_local * ttok + 16 * sub) * ROWB);

  for (int tile = 0; tile < n_tiles; ++tile) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    if (tile + kStages - 1 < n_tiles) issue(tile + kStages - 1);
    cp_async_commit();

    const int wt0 = tok_begin + tile * ttok + 16 * sub;  // first token of this warp's 16
    if (wt0 >= tok_end) continue;                          // warp-uniform: nothing live for this warp
    const uint32_t kbase = smem_base + (uint32_t)((tile % kStages) * STAGE) + warp_rows;
    const uint32_t vbase = kbase + HALF;

    // ---- S = Q K^T over 16 tokens -------------------------------------------------------
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t b[4];
      ldmatrix_x4(b, kbase + k_tl * ROWB + (((2 * kk + k_cx) ^ lr) << 4));
      mma16816<T>(s0, qa[kk], b[0], b[1]);
      mma16816<T>(s1, qa[kk], b[2], b[3]);
    }
    // columns of this thread: tokens wt0 + 2*tg + {0,1} (s0) and + 8 (s1)
    if (wt0 + 16 > tok_end) {
      const int c0 = wt0 + 2 * tg;
      if (c0 >= tok_end) s0[0] = s0[2] = -INFINITY;
      if (c0 + 1 >= tok_end) s0[1] = s0[3] = -INFINITY;
      if (c0 + 8 >= tok_end) s1[0] = s1[2] = -INFINITY;
      if (c0 + 9 >= tok_end) s1[1] = s1[3] = -INFINITY;
    }
    // ---- online softmax on the fragments ------------------------------------------------
    float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    const float mn0 = fmaxf(m0, mx0 * sc);
    float mn1 = m1;
    if (HI) {
      float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      mn1 = fmaxf(m1, mx1 * sc);
    }
    if (__any_sync(0xffffffffu, mn0 > m0 || (HI && mn1 > m1))) {  // rescale only when a row maximum moved
      const float r0 = exp2f(m0 - mn0);                             // m = -inf on first use -> 0
      l0 *= r0;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) { o[j][0] *= r0; o[j][1] *= r0; }
      if (HI) {
        const float r1 = (mn1 == -INFINITY) ? 1.f : exp2f(m1 - mn1);
        l1 *= r1;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) { o[j][2] *= r1; o[j][3] *= r1; }
      }
    }
    m0 = mn0;
    m1 = mn1;
    const float off0 = (mn0 == -INFINITY) ? 0.f : mn0;
    const float p00 = exp2f(fmaf(s0[0], sc, -off0)), p01 = exp2f(fmaf(s0[1], sc, -off0));
    const float p10 = exp2f(fmaf(s1[0], sc, -off0)), p11 = exp2f(fmaf(s1[1], sc, -off0));
    l0 += (p00 + p01) + (p10 + p11);
    uint32_t pa[4];
    pa[0] = pack2<T>(p00, p01);
    pa[2] = pack2<T>(p10, p11);
    pa[1] = pa[3] = 0u;
    if (HI) {
      const float off1 = (mn1 == -INFINITY) ? 0.f : mn1;
      const float q00 = exp2f(fmaf(s0[2], sc, -off1)), q01 = exp2f(fmaf(s0[3], sc, -off1));
      const float q10 = exp2f(fmaf(s1[2], sc, -off1)), q11 = exp2f(fmaf(s1[3], sc, -off1));
      l1 += (q00 + q01) + (q10 + q11);
      pa[1] = pack2<T>(q00, q01);
      pa[3] = pack2<T>(q10, q11);
    }
    // ---- O += P V ---------------------------------------------------------------------------
#pragma unroll
    for (int jn = 0; jn < D / 16; ++jn) {
      uint32_t v[4];
      ldmatrix_x4_trans(v, vbase + v_tl * ROWB + (((2 * jn + v_cx) ^ lr) << 4));
      mma16816<T>(o[2 * jn], pa, v[0], v[1]);
      mma16816<T>(o[2 * jn + 1], pa, v[2], v[3]);
    }
  }
  cp_async_wait<0>();

  // row sums live in quads
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  if (HI) {
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }

  // ---- merge the warps that share a head and write, through shared memory ------------------
  __syncthreads();  // ring no longer read
  constexpr int ROWS = HI ? 16 : 8;
  float* sc_o = reinterpret_cast<float*>(smem);        // [warp][ROWS][D]
  float* sc_ml = sc_o + kWarps * ROWS * D;              // [warp][ROWS][2]
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    *reinterpret_cast<float2*>(&sc_o[(warp * ROWS + g) * D + j * 8 + tg * 2]) = make_float2(o[j][0], o[j][1]);
    if (HI) *reinterpret_cast<float2*>(&sc_o[(warp * ROWS + g + 8) * D + j * 8 + tg * 2]) = make_float2(o[j][2], o[j][3]);
  }
  if (tg == 0) {
    sc_ml[(warp * ROWS + g) * 2] = m0;
    sc_ml[(warp * ROWS + g) * 2 + 1] = l0;
    if (HI) {
      sc_ml[(warp * ROWS + g + 8) * 2] = m1;
      sc_ml[(warp * ROWS + g + 8) * 2 + 1] = l1;
    }
  }
  __syncthreads();

  const int slot = item.w;
  for (int x = tid; x < hb * G * D; x += kThreads) {
    const int d = x % D, r = (x / D) % G, hl = x / (D * G);
    float mx = -INFINITY;
    for (int s2 = 0; s2 < wph; ++s2) mx = fmaxf(mx, sc_ml[(((s2 << hb_log) + hl) * ROWS + r) * 2]);
    float lsum = 0.f, acc = 0.f;
    for (int s2 = 0; s2 < wph; ++s2) {
      const int w2 = (s2 << hb_log) + hl;
      const float mw = sc_ml[(w2 * ROWS + r) * 2];
      const float a = (mw == -INFINITY) ? 0.f : exp2f(mw - mx);
      lsum += sc_ml[(w2 * ROWS + r) * 2 + 1] * a;
      acc += sc_o[(w2 * ROWS + r) * D + d] * a;
    }
    const int qh = (kv_group * hb + hl) * G + r;
    if (slot < 0) {
      const float res = lsum > 0.f ? acc / lsum : 0.f;
      reinterpret_cast<T*>(p.out)[(int64_t)req * p.out_stride + (int64_t)qh * D + d] = from_f32<T>(res);
      if (p.lse != nullptr && d == 0)
        p.lse[(int64_t)req * p.n_q_heads + qh] = lsum > 0.f ? (mx + log2f(lsum)) * 0.6931471805599453f : -INFINITY;
    } else {
      p.part_o[((int64_t)slot * p.n_q_heads + qh) * D + d] = acc;
      if (d == 0) {
        p.part_ml[((int64_t)slot * p.n_q_heads + qh) * 2 + 0] = mx;
        p.part_ml[((int64_t)slot * p.n_q_heads + qh) * 2 + 1] = lsum;
      }
    }
  }
}

}  // namespace mma_decode
}  // namespace dsv
