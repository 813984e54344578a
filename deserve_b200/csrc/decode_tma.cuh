// Paged GQA decode attention for 16-bit K/V with TMA staging.
//
// Same math as decode_mma.cuh (q.K^T and P.V of a GQA group as mma.sync
// m16n8k16 with the group's q heads padded into the 16 A rows, online softmax on
// the fragments with quad shuffles), but the K/V tiles are brought in by the
// Tensor Memory Accelerator: one layer's pages are described to the hardware as
// a 5-D tensor
//     (64 elements, token-in-page, kv head, 64-element half of head_dim, 2*page + {K,V})
// so that ONE cp.async.bulk.tensor instruction gathers the [tokens x heads x
// head_dim] slab of a page into shared memory, token-major per head, with the
// 128-byte hardware swizzle (16-byte chunk index XOR row index mod 8) that makes
// every ldmatrix conflict-free. A ninth warp is the producer: it looks up page
// ids, posts the expected byte count on the stage's "full" mbarrier and issues the
// copies; the eight consumer warps wait on "full", compute, and release the stage
// through its "empty" mbarrier. No thread of the consumers spends an instruction
// on staging. Every wait is bounded: on expiry the kernel records ST_WAIT_TIMEOUT
// in the device status word and returns.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace dsv {
namespace tma_decode {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kStages = 3;
constexpr int kSpinLimit = 1 << 21;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (and a status code) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > (1 << 16)) __nanosleep(64);  // back off only when the wait is clearly not a normal one
  }
  record_status(status, ST_WAIT_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::
          "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

using mma_decode::ldmatrix_x4;
using mma_decode::ldmatrix_x4_trans;
using mma_decode::mma16816;
using mma_decode::pack2;

template <typename T, int D, bool HI>
__global__ void __launch_bounds__(kThreads, 1)
decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
  constexpr int DH = D / 64;            // 64-element halves of head_dim
  constexpr int KSTEPS = D / 16;
  constexpr int HALF = 128 * D * 2;     // K (or V) part of a stage: HB * TTOK = 128 (head, token) rows
  constexpr int STAGE = 2 * HALF;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms are 1024-byte aligned
  unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_full = smem_base + kStages * STAGE;  // kStages x 8 bytes
  const uint32_t bar_empty = bar_full + kStages * 8;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hb_log = p.hb_log2, hb = 1 << hb_log;
  const int wph = kConsumerWarps >> hb_log, ttok = 16 * wph;
  const int ps_log = p.ps_log2, ps = 1 << ps_log;
  const int bt_log = min(ps_log, 4), bt = 1 << bt_log;   // tokens per TMA box
  const int bpg = 16 >> bt_log;                            // boxes per 16-token group
  const int box_bytes = DH * hb * bt * 128;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int kv_group = blockIdx.y;

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

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // ============================ producer warp ============================================
  if (warp == kConsumerWarps) {
    const int32_t* idx = p.kv_indices + ip0;
    const int n_boxes = wph * bpg;          // boxes per tile and per K/V half (<= 16)
    const int sub = lane / bpg, b = lane - sub * bpg;
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % kStages;
      const int tok0 = tok_begin + tile * ttok + 16 * sub + b * bt;  // first token of this lane's box
      const bool mine = lane < n_boxes && tok0 < tok_end;
      int page = 0;
      if (mine) {
        page = __ldg(idx + (tok0 >> ps_log));
        if (page < 0 || page >= p.num_pages) {
          record_status(p.status, ST_BAD_PAGE_ID);
          page = 0;
        }
      }
      if (tile >= kStages) {
        if (!mbar_wait(bar_empty + 8 * s, ((tile / kStages) - 1) & 1, p.status)) return;
      }
      const unsigned live = __ballot_sync(0xffffffffu, mine);
      if (lane == 0) mbar_expect_tx(bar_full + 8 * s, (uint32_t)(__popc(live) * 2 * box_bytes));
      __syncwarp();
      if (mine) {
        const uint32_t dst = smem_base + s * STAGE + (sub * bpg + b) * box_bytes;
        const int in_page = tok0 & (ps - 1);
        tma_load_5d(dst, &tmap, bar_full + 8 * s, 0, in_page, kv_group * hb, 0, 2 * page);
        tma_load_5d(dst + HALF, &tmap, bar_full + 8 * s, 0, in_page, kv_group * hb, 0, 2 * page + 1);
      }
    }
    return;
  }

  // ============================ consumer warps ===========================================
  const int g = lane >> 2, tg = lane & 3;
  const int head_local = warp & (hb - 1), sub = warp >> hb_log;
  const int kv_head = kv_group * hb + head_local;

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
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float sc = p.scale_log2;

  // Row (128 bytes) of token tl of this warp's 16-token group, head head_local, half dh:
  //   ((box * DH + dh) * hb + head_local) * bt + token_in_box, box = tl >> bt_log.
  // ldmatrix lane roles: K matrices (tok lo, c), (tok lo, c+1), (tok hi, c), (tok hi, c+1);
  //                      V matrices (tok lo, c), (tok hi, c), (tok lo, c+1), (tok hi, c+1).
  const int lr = lane & 7, lm = lane >> 3;
  const int k_tl = lr + ((lm >> 1) << 3), k_cx = lm & 1;
  const int v_tl = lr + ((lm & 1) << 3), v_cx = lm >> 1;
  auto row_of = [&](int tl, int dh) { return (((tl >> bt_log) * DH + dh) * hb + head_local) * bt + (tl & (bt - 1)); };
  int k_row[DH], v_row[DH];
#pragma unroll
  for (int dh = 0; dh < DH; ++dh) {
    k_row[dh] = row_of(k_tl, dh);
    v_row[dh] = row_of(v_tl, dh);
  }
  const uint32_t group_off = (uint32_t)(sub * bpg * box_bytes);

  bool ok = true;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    if (!mbar_wait(bar_full + 8 * s, (tile / kStages) & 1, p.status)) {
      ok = false;
      break;
    }
    const int wt0 = tok_begin + tile * ttok + 16 * sub;
    if (wt0 < tok_end) {  // warp-uniform
      const uint32_t kbase = smem_base + s * STAGE + group_off;
      const uint32_t vbase = kbase + HALF;
      const int live = tok_end - wt0;  // live tokens of this group (>= 1)
      if (live < 16) {
        // The copy brought whole boxes: rows of tokens past the end hold whatever the
        // pool holds there. Clear them in V so that 0 * garbage cannot produce a NaN.
        unsigned char* vg = smem + s * STAGE + HALF + group_off;
        for (int x = lane; x < (16 - live) * DH * 8; x += 32) {
          const int ch = x & 7, dh = (x >> 3) % DH, tl = live + (x >> 3) / DH;
          *reinterpret_cast<uint4*>(vg + row_of(tl, dh) * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int cidx = 2 * kk + k_cx, row = k_row[cidx >> 3];
        uint32_t b[4];
        ldmatrix_x4(b, kbase + row * 128 + (((cidx & 7) ^ (row & 7)) << 4));
        mma16816<T>(s0, qa[kk], b[0], b[1]);
        mma16816<T>(s1, qa[kk], b[2], b[3]);
      }
      if (live < 16) {
        const int c0 = 2 * tg;
        if (c0 >= live) s0[0] = s0[2] = -INFINITY;
        if (c0 + 1 >= live) s0[1] = s0[3] = -INFINITY;
        if (c0 + 8 >= live) s1[0] = s1[2] = -INFINITY;
        if (c0 + 9 >= live) s1[1] = s1[3] = -INFINITY;
      }
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
        const float r0 = exp2f(m0 - mn0);
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
#pragma unroll
      for (int jn = 0; jn < D / 16; ++jn) {
        const int cidx = 2 * jn + v_cx, row = v_row[cidx >> 3];
        uint32_t v[4];
        ldmatrix_x4_trans(v, vbase + row * 128 + (((cidx & 7) ^ (row & 7)) << 4));
        mma16816<T>(o[2 * jn], pa, v[0], v[1]);
        mma16816<T>(o[2 * jn + 1], pa, v[2], v[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_empty + 8 * s);  // this warp is done with the stage
  }
  if (!ok) return;

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  if (HI) {
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }

  // ---- merge the warps that share a head and write, through shared memory ------------------
  // every issued copy has been waited for above, so the ring can be reused as scratch
  asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads) : "memory");
  constexpr int ROWS = HI ? 16 : 8;
  float* sc_o = reinterpret_cast<float*>(smem);        // [warp][ROWS][D]
  float* sc_ml = sc_o + kConsumerWarps * ROWS * D;      // [warp][ROWS][2]
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
  asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads) : "memory");

  const int slot = item.w;
  for (int x = tid; x < hb * G * D; x += kConsumerThreads) {
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

// ---- host: the tensor map of one layer's pages ----------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// pages_layer: [P, 2, ps, Hkv, D] 16-bit elements, page stride in elements. Pure host work.
inline bool make_pages_tensor_map(CUtensorMap* map, const void* pages_layer, int64_t page_stride, int64_t num_pages,
                                  int page_size, int n_kv_heads, int head_dim, int hb, bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const int bt = page_size < 16 ? page_size : 16;
  const cuuint64_t half_stride = (cuuint64_t)page_size * n_kv_heads * head_dim * 2;
  if ((cuuint64_t)page_stride * 2 != 2 * half_stride) return false;  // K and V halves must tile the page stride
  const cuuint64_t dims[5] = {64, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, (cuuint64_t)(head_dim / 64),
                              (cuuint64_t)(2 * num_pages)};
  const cuuint64_t strides[4] = {(cuuint64_t)n_kv_heads * head_dim * 2, (cuuint64_t)head_dim * 2, 128, half_stride};
  const cuuint32_t box[5] = {64, (cuuint32_t)bt, (cuuint32_t)hb, (cuuint32_t)(head_dim / 64), 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
            const_cast<void*>(pages_layer), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tma_decode
}  // namespace dsv
