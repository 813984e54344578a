// Ragged causal attention of new q rows against paged K/V (chunked prefill and
// mixed prefill+decode batches) on the 5th-generation tensor cores.
//
// One CTA owns one work item: (request, kv head, two tiles of 128/G q tokens), G =
// n_q_heads / n_kv_heads. The G q heads of the kv head are stacked with the
// tokens into the 128 rows of an MMA (row = token * G + head), so a K/V tile is
// loaded once for the whole GQA group and for both q tiles. Per 128-token K/V
// tile and per q tile:
//     S = Q K^T      tcgen05.mma (kind::f16, M=128, N=128, K=16 x D/16), A and B from
//                    128B-swizzled shared memory, accumulator in TMEM
//     softmax        one warp group per q tile, one thread per row: tcgen05.ld of the row,
//                    causal / length mask, running maximum with lazy rescaling (O is only
//                    rescaled when a row maximum grew by more than 2^8), P = 2^(...) packed to
//                    16 bit and written over S in TMEM with tcgen05.st
//     O += P V       tcgen05.mma with A = P from TMEM and B = the V tile read MN-major
//                    (tokens are the K dimension), accumulator O in TMEM
// The two q tiles ping-pong: while one tile's warp group does its softmax, the tensor
// core runs the other tile's P V and next Q K^T. Warp 8 is the TMA producer of q and
// the K ring (2 stages), warp 10 of the V ring (3 stages: a V slot is released later in
// a tile's life than a K slot and is wanted first in the next one; one
// cp.async.bulk.tensor per 16-token box and 64-element half of head_dim), warp 9 issues the MMAs from one
// thread and signals completion with tcgen05.commit on mbarriers. Every wait is
// bounded; on expiry the kernel records ST_WAIT_TIMEOUT, leaves the loops, frees its
// TMEM and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>
#include <vector>

#include "common.cuh"

namespace dsv {
namespace {

constexpr int kBN = 128;                 // kv tokens per tile
constexpr int kVStages = 3;                // V tiles in flight (K: 2)
constexpr int kThreads = 352;            // 2 x 4 softmax warps, K producer, MMA warp, V producer
constexpr int kSpinLimit = 1 << 21;
constexpr int32_t kPrefillMagic = 0x44535033;  // "DSP3"
// plan header: magic, single-CTA items, q tokens per tile, causal, batch, offset of the single-CTA items,
// q heads, kv heads, pair items, offset of the pair items, 2 unused; then the items, 4 int32 each
constexpr int kPlanHeader = 12;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;  // log2 units

struct PrefillParams {
  const int32_t* qo_indptr;
  const int32_t* kv_indices;
  const int32_t* kv_indptr;
  const int32_t* kv_last_page_len;
  void* out;
  const int4* items;  // {request, first q token of the tile (request-relative), q tokens in the tile, visible kv length of its last token}
  int64_t out_stride;
  int n_q_heads, n_kv_heads, ps_log2, num_pages, causal;
  float scale_log2;
  int* status;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > (1 << 16)) __nanosleep(64);  // back off only when the wait is clearly not a normal one
  }
  record_status(status, ST_WAIT_TIMEOUT);
  return false;
}
// The same wait made warp-uniform: every lane leaves with the same answer, so the
// warp-collective tcgen05 instructions that follow are executed by all lanes or by none.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int* status) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, status));
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::
          "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::
          "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the same two with the accumulate flag fixed to "add to D": no predicate set-up per instruction
__device__ __forceinline__ void umma_ss_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, 1;\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
               "r"(idesc)
               : "memory");
}
__device__ __forceinline__ void umma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile("tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 1;\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc),
               "r"(idesc)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version field.
// K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO); LBO unused (1).
// MN-major: 64-element blocks of the MN dimension `lbo_bytes` apart, 8-row groups of the
// K dimension 1024 bytes apart (SBO).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: fp32 accumulate, A/B format (0 = f16, 1 = bf16),
// B major-ness (0 = K, 1 = MN), N >> 3, M >> 4.
__host__ __device__ constexpr uint32_t instr_desc(int ab_format, int b_mn_major, int n, int m) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float ex2(float x) {  // 2^x on the special-function unit; ex2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32 pairs: one instruction for two columns of a row. The softmax warps are bound by how
// many instructions they issue per score, not by the special-function unit alone.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n .reg .b64 a, b, c, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n mov.b64 c, {%6, %7};\n"
      " fma.rn.f32x2 d, a, b, c;\n mov.b64 {%0, %1}, d;\n}\n"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n .reg .b64 a, b, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n add.rn.f32x2 d, a, b;\n mov.b64 {%0, %1}, d;\n}\n"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
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

// ---- the kernel ---------------------------------------------------------------------------------
// Warp roles: 0-3 softmax of q tile A, 4-7 softmax of q tile B (thread = row = TMEM lane), 8 TMA
// producer of q and the K ring, 9 MMA issuer, 10 TMA producer of the V ring.
// TMEM columns: tile X owns [256 X, 256 X + 256): S at +0 (P is written over its first 64 columns
// once the row has been read), O at +128.
// MERGED (head_dim 128, pages of 16 tokens or more): a K/V box is 16 tokens x both 64-element halves of
// head_dim, 4 KB instead of two boxes of 2 KB. The K/V feed is bound by the number of TMA boxes an SM can
// issue (80-100 cycles each at 2 KB, 110-135 at 4 KB, whatever their rank), not by their bytes. K boxes
// come through k_map, which splits the token index so that a box lands as [8-token group][half][8 tokens]
// [128 B]: 8-token groups 2 KB apart for either half, which one K-major descriptor walks. V boxes come
// through v_map as [half][16 tokens][128 B]; a 16-token step of P V is one box, halves 2 KB apart.
template <typename T, int D, bool MERGED>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
               const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
               const PrefillParams p) {
  constexpr int DH = D / 64;
  constexpr int QTILE = 128 * D * 2;      // one q tile: [DH][128 rows][128 B]
  constexpr int KVTILE = kBN * D * 2;     // one K (or V) stage: [DH][128 tokens][128 B]
  constexpr int HALF_ROWS = 128 * 128;    // bytes of one 64-element half: 128 rows x 128 B
  static_assert(!MERGED || D == 128, "merged boxes hold both halves of a 128-element head");
  // K stage: [DH][128 tokens][128 B], or merged [16 groups][DH][8 tokens][128 B]
  constexpr int K_GROUP = MERGED ? 2048 : 1024;     // bytes between 8-token groups of one half
  constexpr int K_HALF = MERGED ? 1024 : HALF_ROWS; // bytes between the halves of head_dim
  // V stage: [DH][128 tokens][128 B], or merged [8 boxes][DH][16 tokens][128 B]
  constexpr int V_STEP = MERGED ? 4096 : 2048;      // bytes between 16-token steps
  constexpr int V_HALF = MERGED ? 2048 : HALF_ROWS;
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr uint32_t IDESC_QK = instr_desc(kBf16 ? 1 : 0, 0, kBN, 128);
  constexpr uint32_t IDESC_PV = instr_desc(kBf16 ? 1 : 0, 1, D, 128);
  constexpr uint32_t COL_S = 0, COL_O = 128, COL_TILE = 256;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;                       // 2 q tiles
  const uint32_t k_smem = q_smem + 2 * QTILE;         // 2 stages
  const uint32_t v_smem = k_smem + 2 * KVTILE;        // kVStages stages
  const uint32_t bars = v_smem + kVStages * KVTILE;
  // barrier slots (8 bytes each): q, kfull[2], vfull[3], kempty[2], vempty[3], sfull[2 tiles], pfull[2], odone[2]
  const uint32_t bar_q = bars, bar_kfull = bars + 8, bar_vfull = bars + 24, bar_kempty = bars + 48,
                 bar_vempty = bars + 64, bar_sfull = bars + 88, bar_pfull = bars + 104, bar_odone = bars + 120;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + (bars - base) + 136);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int tq = 128 / G;                  // q tokens per tile
  // consecutive CTAs are the kv heads of one item: together they read whole token rows of the same pages
  const int kv_head = blockIdx.x % p.n_kv_heads;
  const int ps_log = p.ps_log2, ps = 1 << ps_log;
  const int bt = min(ps, 16), n_boxes = kBN / bt;

  const int4 item = p.items[blockIdx.x / p.n_kv_heads];
  const int req = item.x, q0 = item.y, nq = item.z, kv_hi = item.w;
  const int q_begin = __ldg(p.qo_indptr + req);
  const int n_new = __ldg(p.qo_indptr + req + 1) - q_begin;
  const int ip0 = __ldg(p.kv_indptr + req), ip1 = __ldg(p.kv_indptr + req + 1);
  const int kv_len = ip1 > ip0 ? (ip1 - ip0 - 1) * ps + __ldg(p.kv_last_page_len + req) : 0;
  const int n_tiles = (kv_hi + kBN - 1) / kBN;
  const bool has_b = nq > tq;              // the second q tile holds live rows
  const bool bad = q0 < 0 || nq < 1 || nq > 2 * tq || q0 + nq > n_new || kv_hi < 1 || kv_hi > kv_len;
  if (bad) {
    if (tid == 0) record_status(p.status, ST_BAD_PLAN);
    return;
  }

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_pfull + 8 * s, 4);  // one arrival per softmax warp
      mbar_init(bar_odone + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 8) {  // TMEM: all 512 columns (one CTA per SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(const_cast<uint32_t*>(tmem_slot))),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8 || warp == 10) {
    // ================================ TMA producers: warp 8 = q + K ring, warp 10 = V ring =======
    if (warp == 8 && lane == 0) {
      mbar_expect_tx(bar_q, (uint32_t)(QTILE * (has_b ? 2 : 1)));
      for (int x = 0; x < (has_b ? 2 : 1); ++x)
        for (int dh = 0; dh < DH; ++dh)
          tma_load_4d(q_smem + x * QTILE + dh * HALF_ROWS, &q_map, bar_q, 0, kv_head * G, dh, q_begin + q0 + x * tq);
    }
    const int32_t* idx = p.kv_indices + ip0;
    const int kv = warp == 10 ? 1 : 0;
    const int n_stages = kv ? kVStages : 2;
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int s = tile % n_stages, round = tile / n_stages;
      const int t0 = tile * kBN;
      int live = 0;  // boxes that hold at least one visible token
      for (int b = 0; b < n_boxes; ++b) live += (t0 + b * bt < kv_hi) ? 1 : 0;
      // The K and V rings advance on their own barriers and in their own warps: a K stage is free
      // as soon as Q K^T of two tiles ago has run, so the next K tile is in flight long before the
      // MMA warp asks for it, whatever the V ring is waiting for.
      const uint32_t full = (kv ? bar_vfull : bar_kfull) + 8 * s, empty = (kv ? bar_vempty : bar_kempty) + 8 * s;
      if (round > 0 && !warp_wait(empty, (round - 1) & 1, p.status)) break;
      if (lane == 0) mbar_expect_tx(full, (uint32_t)(live * DH * bt * 128));
      __syncwarp();
      for (int b = lane; b < n_boxes; b += 32) {
        const int tok = t0 + b * bt;
        if (tok >= kv_hi) continue;
        int page = __ldg(idx + (tok >> ps_log));
        if (page < 0 || page >= p.num_pages) {
          record_status(p.status, ST_BAD_PAGE_ID);
          page = 0;
        }
        const int in_page = tok & (ps - 1);
        if constexpr (MERGED) {  // bt = 16: one 4 KB box per 16 tokens
          const uint32_t dst = (kv ? v_smem : k_smem) + (uint32_t)(s * KVTILE + b * 4096);
          if (kv) tma_load_5d(dst, &v_map, full, 0, in_page, kv_head, 0, 2 * page + 1);
          else tma_load_5d(dst, &k_map, full, 0, 0, 2 * kv_head, in_page >> 3, 2 * page);
        } else {
          for (int dh = 0; dh < DH; ++dh) {
            const uint32_t off = (uint32_t)(s * KVTILE + dh * HALF_ROWS + b * bt * 128);
            tma_load_5d((kv ? v_smem : k_smem) + off, &kv_map, full, 0, in_page, kv_head, dh, 2 * page + kv);
          }
        }
      }
    }
  } else if (warp == 9) {
    // ================================ MMA issuer (one thread) ===================================
    // Issue order per K/V tile j: P_A V, next Q_A K^T, P_B V, next Q_B K^T. While the softmax warps
    // of one q tile work, the tensor core runs the other tile's two products.
    if (lane == 0) {
      bool ok = mbar_wait(bar_q, 0, p.status);
      // Matrix descriptors are built once; inside the loops a descriptor is one 64-bit add of a
      // compile-time offset (the start-address field counts 16-byte units). The issuing thread is a
      // single lane: every instruction it spends per MMA is on the critical path of the tensor core.
      const uint64_t qd[2] = {smem_desc(q_smem, 16, 1024), smem_desc(q_smem + QTILE, 16, 1024)};
      const uint64_t kd[2] = {smem_desc(k_smem, 16, K_GROUP), smem_desc(k_smem + KVTILE, 16, K_GROUP)};
      const uint64_t vd0 = smem_desc(v_smem, V_HALF, 1024);
      auto issue_qk = [&](int tile, int x) {  // S_x = Q_x K_tile^T
        const int s = tile & 1;
        const uint32_t d = tmem + x * COL_TILE + COL_S;
        const uint64_t qa = qd[x], kb = kd[s];
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr int kUnit = 16;  // bytes per descriptor address unit
          const uint64_t qoff = (uint64_t)(((kk >> 2) * HALF_ROWS + (kk & 3) * 32) / kUnit);
          const uint64_t koff = (uint64_t)(((kk >> 2) * K_HALF + (kk & 3) * 32) / kUnit);
          if (kk == 0) umma_ss(d, qa + qoff, kb + koff, IDESC_QK, 0u);
          else umma_ss_acc(d, qa + qoff, kb + koff, IDESC_QK);
        }
        tc_commit(bar_sfull + 8 * x);
        if (x == (has_b ? 1 : 0)) tc_commit(bar_kempty + 8 * s);  // last reader of this K stage
      };
      auto issue_pv = [&](int tile, int x) {  // O_x += P_x V_tile
        const int s = tile % kVStages;
        const int cols = min(kBN, kv_hi - tile * kBN);
        const int ksteps = (cols + 15) >> 4;  // 16-token steps that hold a visible token
        const uint32_t d = tmem + x * COL_TILE + COL_O, a = tmem + x * COL_TILE + COL_S;
        const uint64_t vb = vd0 + (uint64_t)(s * (KVTILE / 16));
        if (ksteps == kBN / 16 && tile > 0) {  // the common case, fully unrolled
#pragma unroll
          for (int kt = 0; kt < kBN / 16; ++kt) umma_ts_acc(d, a + kt * 8, vb + (uint64_t)(kt * V_STEP / 16), IDESC_PV);
        } else {
          for (int kt = 0; kt < ksteps; ++kt)
            umma_ts(d, a + kt * 8, vb + (uint64_t)(kt * V_STEP / 16), IDESC_PV, (tile > 0 || kt > 0) ? 1u : 0u);
        }
        tc_commit(bar_odone + 8 * x);
        if (x == (has_b ? 1 : 0)) tc_commit(bar_vempty + 8 * s);  // last reader of this V stage
      };
      if (ok) ok = mbar_wait(bar_kfull, 0, p.status);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        if (has_b) issue_qk(0, 1);
      }
      for (int tile = 0; ok && tile < n_tiles; ++tile) {
        const int s = tile & 1;
        const bool more = tile + 1 < n_tiles;
        // This tile's V and the next tile's K landed long ago (the rings run ahead): look at their
        // barriers now, while the softmax warps are still busy, not between two products.
        ok = mbar_wait(bar_vfull + 8 * (tile % kVStages), (tile / kVStages) & 1, p.status);
        if (ok && more) ok = mbar_wait(bar_kfull + 8 * (s ^ 1), ((tile + 1) >> 1) & 1, p.status);
        for (int x = 0; ok && x < (has_b ? 2 : 1); ++x) {
          ok = mbar_wait(bar_pfull + 8 * x, tile & 1, p.status);
          if (!ok) break;
          tc_fence_after();
          issue_pv(tile, x);
          if (more) {
            issue_qk(tile + 1, x);  // runs after P_x V (in issue order), so S_x / P_x may be overwritten
          }
        }
      }
    }
  } else {
    // ================================ softmax / correction / epilogue ============================
    const int x = warp >> 2;                  // q tile of this warp group
    const int row = tid & 127;                // TMEM lane and MMA row
    if (x == 0 || has_b) {
      const int tok_local = x * tq + row / G, head = row % G;
      const bool row_live = tok_local < nq;
      // last kv position this row may see
      const int limit = min(p.causal ? (kv_len - n_new + q0 + tok_local) : (kv_len - 1), kv_hi - 1);
      const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
      const uint32_t s_addr = tmem + lane_base + x * COL_TILE + COL_S;
      const uint32_t o_addr = tmem + lane_base + x * COL_TILE + COL_O;
      const float sc = p.scale_log2;
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      for (int tile = 0; tile < n_tiles; ++tile) {
        if (!warp_wait(bar_sfull + 8 * x, tile & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const int t0 = tile * kBN;
        const bool need_mask = (t0 + kBN - 1) > limit;
        // the whole S row in registers: four 32-column loads in flight, one wait
        uint32_t r[kBN];
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_wait_ld();
        float mx = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < kBN; ++i)
            if (t0 + i > limit) r[i] = 0xff800000u;  // -inf
        }
        {  // eight independent chains of three-input maxima instead of one 128-long dependent chain
          float m8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) m8[i] = __uint_as_float(r[i]);
#pragma unroll
          for (int i = 8; i + 15 < kBN; i += 16) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              m8[j] = fmax3(m8[j], __uint_as_float(r[i + 2 * j]), __uint_as_float(r[i + 2 * j + 1]));
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) m8[j] = fmaxf(m8[j], __uint_as_float(r[kBN - 8 + j]));  // 8 + 7 * 16 = 120 done
          mx = fmaxf(fmax3(m8[0], m8[1], m8[2]), fmaxf(fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
        }
        const float m_tile = mx * sc;
        // lazy rescale: keep the old reference maximum unless the row maximum grew by more than 2^8
        float factor = 1.f;
        if (m_tile > m_used + kRescaleThreshold || (m_used == -INFINITY && m_tile > -INFINITY)) {
          factor = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_tile);
          m_used = m_tile;
        }
        if (tile > 0) {
          // O is free: S of this tile was issued behind the previous P V and completions are in
          // issue order, so seeing this S means that P V has finished. No wait needed.
          if (__any_sync(0xffffffffu, factor != 1.f)) {
            l *= factor;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(o_addr + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_st32(o_addr + c * 32, o);
            }
          }
        }
        // P = 2^(S * scale - m_used) (masked entries give 2^-inf = 0), written over S as 16-bit pairs
        const float off = (m_used == -INFINITY) ? 0.f : m_used;
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1, a, b;
            ffma2(x0, x1, __uint_as_float(r[c * 32 + 2 * i]), __uint_as_float(r[c * 32 + 2 * i + 1]), sc, sc, -off, -off);
            a = ex2(x0);
            b = ex2(x1);
            fadd2(ls[2 * (i & 1)], ls[2 * (i & 1) + 1], ls[2 * (i & 1)], ls[2 * (i & 1) + 1], a, b);
            pk[i] = pack2<T>(a, b);
          }
          tmem_st16(s_addr + c * 16, pk);
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        tmem_wait_st();
        // Rows of V past the visible length hold whatever the pool (or an older tile) left there;
        // clear the ones inside the last issued 16-token step so that 0 * garbage stays 0. Both
        // warp groups write the same zeros; each does it before releasing its own P.
        const int cols = min(kBN, kv_hi - t0);
        if (cols < kBN && (cols & 15) != 0) {
          const int vs = tile % kVStages;
          if (!warp_wait(bar_vfull + 8 * vs, (tile / kVStages) & 1, p.status)) { ok = false; break; }
          const int r0 = cols, r1 = (cols + 15) & ~15;
          for (int z = row; z < (r1 - r0) * DH * 8; z += 128) {
            const int ch = z & 7, dh = (z >> 3) % DH, rr = r0 + (z >> 3) / DH;
            const int at = MERGED ? (rr >> 4) * V_STEP + dh * V_HALF + (rr & 15) * 128 : dh * HALF_ROWS + rr * 128;
            *reinterpret_cast<uint4*>(smem + (v_smem - base) + vs * KVTILE + at + ch * 16) = make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pfull + 8 * x);
      }
      if (ok) ok = warp_wait(bar_odone + 8 * x, (n_tiles - 1) & 1, p.status);
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* dst = reinterpret_cast<T*>(p.out) + (int64_t)(q_begin + q0 + tok_local) * p.out_stride +
                 (int64_t)(kv_head * G + head) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
          if (row_live) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i)
                w[i] = pack2<T>(__uint_as_float(o[v * 8 + 2 * i]) * inv, __uint_as_float(o[v * 8 + 2 * i + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }
  }

  // ---- teardown: everyone meets here, then the allocating warp frees TMEM ----------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---- the pair kernel: two CTAs of a cluster on one K/V stream ---------------------------------------
// A cluster of two CTAs (cta_group::2) owns (request, kv head, two q tiles of 128/G tokens), one q
// tile per CTA. One MMA covers both tiles (M = 256: rows 0-127 in CTA 0's TMEM, 128-255 in CTA 1's),
// so a K/V block feeds two q tiles while each CTA loads and holds only half of it: for S = Q K^T
// (N = 128 kv tokens) CTA c holds tokens [64c, 64c+64) of the block, for O += P V (N = head_dim) it
// holds the 64-element half c of head_dim. Per SM that is the K/V traffic of prefill_kernel (one
// block per two q tiles) with half the B-operand reads from shared memory.
//
// With one q tile per CTA the 512 TMEM columns hold S twice (S0 at 0, S1 at 128), O (at 256) and
// P twice (P0 at 384, P1 at 448). The two softmax warp groups take alternate K/V blocks: group a
// works on the blocks j = a (mod 2). It gives S_a back as soon as the row is in registers, so Q K^T
// of block j+2 runs while the group is still busy with block j and S is there when it comes back;
// P_j goes to P_a, which P V of block j reads while the group already works on block j+2. Neither
// group waits for the tensor core in steady state, and the special-function unit sees the two
// groups half a block apart. What the groups share per row is the reference maximum of the lazily rescaled
// softmax: the group of block j reads the reference left by block j-1 (shared memory, a named
// barrier per warp pair), raises it if its own row maximum is more than 2^8 above it, and publishes
// it; only the group that raises it rescales O (after P V of block j-1 has finished), and each group
// brings its own partial row sum to the current reference when it next sees it.
//
// Two threads of CTA 0 issue the MMAs: warp 9 the Q K^T products, warp 11 the P V products.
// Barriers those threads wait on (q, kfull, vfull, sfree, pfull) live in CTA 0 and are signalled by
// both CTAs (TMA complete_tx through the cta_group::2 form, remote arrives); barriers the other
// warps wait on (kempty, vempty, sfull, pvdone) exist in both CTAs and are committed to in both.
// Every wait is bounded; both CTAs meet at a cluster barrier before the TMEM is freed.
constexpr int kPairThreads = 384;  // 2 x 4 softmax warps, q + K producer, Q K^T issuer, V producer, P V issuer
constexpr int kPKStages = 6;       // K blocks in flight (a load takes several block times to arrive)
constexpr int kPVStages = 5;       // V blocks in flight

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {  // shared::cta -> shared::cluster of `rank`
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Arrivals on a barrier of any CTA of the cluster (address from map_to_cta). The plain form orders
// nothing but the tensor-memory traffic that tcgen05.wait and tcgen05.fence have already closed; the
// release form (hundreds of cycles) is for shared-memory writes the waiting side reads.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA loads of a CTA pair: the data lands in this CTA, the bytes are counted on `bar`, which may be
// the peer's barrier
__device__ __forceinline__ void tma2_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                             int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::
          "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma2_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::
          "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// completion of the MMAs issued so far by this thread: one arrival on the barrier at this offset in
// each of the two CTAs
__device__ __forceinline__ void tc2_commit_both(uint32_t bar_cluster) {
  asm volatile(
      "{\n .reg .b16 m;\n mov.b16 m, 3;\n"
      " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n}\n" ::"r"(
          bar_cluster)
      : "memory");
}
__device__ __forceinline__ void umma2_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_ss_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile("tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, 1;\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc),
               "r"(idesc)
               : "memory");
}
__device__ __forceinline__ void umma2_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma2_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile("tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, 1;\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc),
               "r"(idesc)
               : "memory");
}
// two barriers in one polling loop (a satisfied wait costs a few hundred cycles: pay it once)
__device__ __forceinline__ bool warp_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b,
                                           int* status) {
  bool done = false;
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar_a, parity_a) && mbar_try_wait(bar_b, parity_b)) {
      done = true;
      break;
    }
    if (i > (1 << 16)) __nanosleep(64);
  }
  if (!done) record_status(status, ST_WAIT_TIMEOUT);
  return __all_sync(0xffffffffu, done);
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// Warp roles: 0-3 softmax of the even K/V blocks, 4-7 of the odd ones (thread = row = TMEM lane),
// 8 TMA producer of q and the K ring, 9 Q K^T issuer (CTA 0), 10 TMA producer of the V ring,
// 11 P V issuer (CTA 0).
template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                    const __grid_constant__ CUtensorMap k_map, const PrefillParams p) {
  constexpr int D = 128, DH = 2;
  constexpr int QTILE = 128 * D * 2;        // the q tile: [DH][128 rows][128 B]
  // this CTA's 64 tokens of a K block: [8-token group][half of head_dim][8 tokens][128 B]. One TMA box
  // is 16 tokens x both halves (4 KB; the issue rate of TMA boxes, not their bytes, bounds the K/V feed).
  constexpr int KGROUP = DH * 8 * 128;      // 2 KB
  constexpr int KSTAGE = 8 * KGROUP;
  constexpr int VSTAGE = kBN * 128;         // [128 tokens][128 B]: this CTA's 64-element half of head_dim
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr uint32_t IDESC_QK = instr_desc(kBf16 ? 1 : 0, 0, kBN, 256);
  constexpr uint32_t IDESC_PV = instr_desc(kBf16 ? 1 : 0, 1, D, 256);
  constexpr uint32_t COL_O = 256, COL_P = 384;  // S0 at 0, S1 at 128; P0 at 384, P1 at 448

  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem = q_smem + QTILE;
  const uint32_t v_smem = k_smem + kPKStages * KSTAGE;
  const uint32_t f_smem = v_smem + kPVStages * VSTAGE;     // floats: mref[2][128], lsum[2][128], mfin[2][128]
  const uint32_t bars = f_smem + 6 * 128 * 4;
  float* fl = reinterpret_cast<float*>(smem + (f_smem - base));
  float* mref = fl;             // [group][row]: the reference maximum after that group's latest block
  float* lsum = fl + 256;       // [group][row]: partial row sums, for the epilogue
  float* mfin = fl + 512;       // [group][row]: the reference each partial sum is scaled to
  // barrier slots (8 bytes each)
  constexpr uint32_t B_Q = 0, B_KFULL = 1, B_VFULL = B_KFULL + kPKStages, B_KEMPTY = B_VFULL + kPVStages,
                     B_VEMPTY = B_KEMPTY + kPKStages, B_SFULL = B_VEMPTY + kPVStages, B_PFULL = B_SFULL + 2,
                     B_PVDONE = B_PFULL + 2, B_SFREE = B_PVDONE + 2, B_VLAST = B_SFREE + 2, B_MREF = B_VLAST + 1,
                     B_COUNT = B_MREF + 8;  // mref: [group][warp of the group], one arrival per published block
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + (bars - base) + 8 * B_COUNT);
  auto bar = [&](uint32_t slot) { return bars + 8 * slot; };

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  const int G = p.n_q_heads / p.n_kv_heads;
  const int tq = 128 / G;                  // q tokens per tile
  // consecutive clusters are the kv heads of one item: together they read whole token rows of the same pages
  const int kv_head = (blockIdx.x >> 1) % p.n_kv_heads;
  const int ps_log = p.ps_log2, ps = 1 << ps_log;
  const int bt = min(ps, 16);

  const int4 item = p.items[(blockIdx.x >> 1) / p.n_kv_heads];
  const int req = item.x, q0 = item.y, nq = item.z, kv_hi = item.w;
  const int q_begin = __ldg(p.qo_indptr + req);
  const int n_new = __ldg(p.qo_indptr + req + 1) - q_begin;
  const int ip0 = __ldg(p.kv_indptr + req), ip1 = __ldg(p.kv_indptr + req + 1);
  const int kv_len = ip1 > ip0 ? (ip1 - ip0 - 1) * ps + __ldg(p.kv_last_page_len + req) : 0;
  const int n_blocks = (kv_hi + kBN - 1) / kBN;
  // the same verdict in both CTAs of the pair: both leave before any cluster-wide step
  const bool bad = q0 < 0 || nq < 1 || nq > 2 * tq || q0 + nq > n_new || kv_hi < 1 || kv_hi > kv_len;
  if (bad) {
    if (tid == 0) record_status(p.status, ST_BAD_PLAN);
    return;
  }

  if (tid == 0) {
    mbar_init(bar(B_Q), 2);  // one arrival (with its byte count) per CTA
    for (int s = 0; s < kPKStages; ++s) {
      mbar_init(bar(B_KFULL + s), 2);
      mbar_init(bar(B_KEMPTY + s), 1);
    }
    for (int s = 0; s < kPVStages; ++s) {
      mbar_init(bar(B_VFULL + s), 2);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(B_SFULL + s), 1);
      mbar_init(bar(B_PFULL + s), 8);  // one arrival per warp of the softmax group, both CTAs
      mbar_init(bar(B_SFREE + s), 8);
      mbar_init(bar(B_PVDONE + s), 1);
    }
    mbar_init(bar(B_VLAST), 1);
    for (int s = 0; s < 8; ++s) mbar_init(bar(B_MREF + s), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 8) {  // TMEM: all 512 columns of both SMs; the same warp of both CTAs takes part
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(const_cast<uint32_t*>(tmem_slot))),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lead = map_to_cta(bars, 0) - bars;  // add to a local barrier address: the same barrier in CTA 0

  if (warp == 8) {
    // ================================ q and the K ring ==========================================
    if (lane == 0) {
      mbar_expect_tx_cluster(bar(B_Q) + lead, (uint32_t)QTILE);
      for (int dh = 0; dh < DH; ++dh)
        tma2_load_4d(q_smem + dh * (128 * 128), &q_map, bar(B_Q) + lead, 0, kv_head * G, dh,
                     q_begin + q0 + (int)rank * tq);
    }
    // One TMA per lane and 16-token box. The page id of the next block's box is fetched while this
    // block's loads are issued: a producer that looks up the page table inside the step is slower
    // than the block time of the rest of the kernel.
    const int32_t* idx = p.kv_indices + ip0;
    auto page_of = [&](int tok) -> int {
      if (tok >= kv_hi) return -1;  // nothing to load
      int page = __ldg(idx + (tok >> ps_log));
      if (page < 0 || page >= p.num_pages) {
        record_status(p.status, ST_BAD_PAGE_ID);
        page = 0;
      }
      return page;
    };
    const int tok_lane = (int)rank * 64 + lane * 16;  // first token of this lane's box in block 0
    int page_next = lane < 4 ? page_of(tok_lane) : -1;
    int s = 0;
    uint32_t parity = 1;  // the parity of "stage never used": the first pass over the ring does not wait
    for (int j = 0; j < n_blocks; ++j) {
      const int t0 = j * kBN + (int)rank * 64;  // this CTA's 64 tokens of the block
      const int live = min(4, max(0, (kv_hi - t0 + 15) / 16));  // boxes that hold a visible token
      const int page_now = page_next;
      if (j + 1 < n_blocks && lane < 4) page_next = page_of(tok_lane + (j + 1) * kBN);
      if (j >= kPKStages && !warp_wait(bar(B_KEMPTY + s), parity, p.status)) break;
      if (lane == 0) mbar_expect_tx_cluster(bar(B_KFULL + s) + lead, (uint32_t)(live * 2 * KGROUP));
      __syncwarp();
      if (lane < 4 && page_now >= 0) {
        const int tok = t0 + lane * 16;
        // coordinates: element, token within its group of 8, head * 2 + half, group of 8 within the page, 2 * page + {K, V}
        tma2_load_5d(k_smem + (uint32_t)(s * KSTAGE + lane * 2 * KGROUP), &k_map, bar(B_KFULL + s) + lead, 0, 0, 2 * kv_head,
                     (tok & (ps - 1)) >> 3, 2 * page_now);
      }
      if (++s == kPKStages) {
        s = 0;
        parity ^= 1;
      }
    }
  } else if (warp == 10) {
    // ================================ the V ring: this CTA's half of head_dim ====================
    const int32_t* idx = p.kv_indices + ip0;
    const int units = kBN / bt;  // one TMA per lane, page ids fetched one block ahead (see the K ring)
    auto page_of = [&](int tok) -> int {
      if (tok >= kv_hi) return -1;
      int page = __ldg(idx + (tok >> ps_log));
      if (page < 0 || page >= p.num_pages) {
        record_status(p.status, ST_BAD_PAGE_ID);
        page = 0;
      }
      return page;
    };
    int page_next = lane < units ? page_of(lane * bt) : -1;
    int s = 0;
    uint32_t parity = 1;
    for (int j = 0; j < n_blocks; ++j) {
      const int t0 = j * kBN;
      const int cols = min(kBN, kv_hi - t0);
      // Rows past the visible length inside the last 16-token step hold whatever the pool left
      // there; 0 * garbage must stay 0, so that block goes through a local barrier, the rows are
      // cleared, and the arrival on CTA 0's barrier is a plain one.
      const bool ragged = (cols & 15) != 0;
      const int live = (cols + bt - 1) / bt;
      const int page_now = page_next;
      if (j + 1 < n_blocks && lane < units) page_next = page_of((j + 1) * kBN + lane * bt);
      if (j >= kPVStages && !warp_wait(bar(B_VEMPTY + s), parity, p.status)) break;
      const uint32_t full = ragged ? bar(B_VLAST) : bar(B_VFULL + s) + lead;
      if (lane == 0) {
        if (ragged) mbar_expect_tx(full, (uint32_t)(live * bt * 128));
        else mbar_expect_tx_cluster(full, (uint32_t)(live * bt * 128));
      }
      __syncwarp();
      for (int u = lane; u < units; u += 32) {
        const int tok = t0 + u * bt;
        const int page = u < 32 ? page_now : page_of(tok);
        if (page < 0) continue;
        tma2_load_5d(v_smem + (uint32_t)(s * VSTAGE + u * bt * 128), &kv_map, full, 0, tok & (ps - 1), kv_head, (int)rank,
                     2 * page + 1);
      }
      if (ragged) {  // only the last block of the item can be ragged: the local barrier is used once
        if (!warp_wait(bar(B_VLAST), 0, p.status)) break;
        const int r0 = cols, r1 = (cols + 15) & ~15;
        for (int z = lane; z < (r1 - r0) * 8; z += 32)
          *reinterpret_cast<uint4*>(smem + (v_smem - base) + s * VSTAGE + (r0 + (z >> 3)) * 128 + (z & 7) * 16) =
              make_uint4(0, 0, 0, 0);
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_release(bar(B_VFULL + s) + lead);
      }
      if (++s == kPVStages) {
        s = 0;
        parity ^= 1;
      }
    }
  } else if (warp == 9) {
    // ================================ Q K^T issuer: one thread of CTA 0 ==========================
    if (rank == 0 && lane == 0) {
      bool ok = mbar_wait(bar(B_Q), 0, p.status);
      const uint64_t qd = smem_desc(q_smem, 16, 1024);
      const uint64_t kd0 = smem_desc(k_smem, 16, KGROUP);  // 8-token groups 2 KB apart
      int s = 0;
      uint32_t parity = 0;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int a = j & 1;
        ok = mbar_wait(bar(B_KFULL + s), parity, p.status);
        // S_a is free once its group has block j-2 in registers
        if (ok && j >= 2) ok = mbar_wait(bar(B_SFREE + a), ((j - 2) >> 1) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem + a * kBN;
        const uint64_t kb = kd0 + (uint64_t)(s * (KSTAGE / 16));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t qoff = (uint64_t)(((kk >> 2) * (128 * 128) + (kk & 3) * 32) / 16);
          const uint64_t koff = (uint64_t)(((kk >> 2) * (8 * 128) + (kk & 3) * 32) / 16);
          if (kk == 0) umma2_ss(d, qd + qoff, kb + koff, IDESC_QK, 0u);
          else umma2_ss_acc(d, qd + qoff, kb + koff, IDESC_QK);
        }
        tc2_commit_both(bar(B_SFULL + a));
        tc2_commit_both(bar(B_KEMPTY + s));
        if (++s == kPKStages) {
          s = 0;
          parity ^= 1;
        }
      }
    }
  } else if (warp == 11) {
    // ================================ P V issuer: one thread of CTA 0 ============================
    if (rank == 0 && lane == 0) {
      const uint64_t vd0 = smem_desc(v_smem, VSTAGE, 1024);
      bool ok = true;
      int s = 0;
      uint32_t parity = 0;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int a = j & 1;
        ok = mbar_wait(bar(B_VFULL + s), parity, p.status);
        if (ok) ok = mbar_wait(bar(B_PFULL + a), (j >> 1) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        const int cols = min(kBN, kv_hi - j * kBN);
        const int ksteps = (cols + 15) >> 4;  // 16-token steps that hold a visible token
        const uint32_t d = tmem + COL_O, pa = tmem + COL_P + a * (kBN / 2);
        const uint64_t vb = vd0 + (uint64_t)(s * (VSTAGE / 16));
        if (ksteps == kBN / 16 && j > 0) {  // the common case, fully unrolled
#pragma unroll
          for (int kt = 0; kt < kBN / 16; ++kt) umma2_ts_acc(d, pa + kt * 8, vb + (uint64_t)(kt * 2048 / 16), IDESC_PV);
        } else {
          for (int kt = 0; kt < ksteps; ++kt)
            umma2_ts(d, pa + kt * 8, vb + (uint64_t)(kt * 2048 / 16), IDESC_PV, (j > 0 || kt > 0) ? 1u : 0u);
        }
        tc2_commit_both(bar(B_PVDONE + a));  // P_a is free, O holds block j
        tc2_commit_both(bar(B_VEMPTY + s));
        if (++s == kPVStages) {
          s = 0;
          parity ^= 1;
        }
      }
    }
  } else {
    // ================================ softmax / correction / epilogue ============================
    const int a = warp >> 2;                  // this group's blocks: j = a (mod 2), in S_a
    const int row = tid & 127;                // TMEM lane and MMA row
    const int tok_local = (int)rank * tq + row / G, head = row % G;
    const bool row_live = tok_local < nq;
    const int limit = min(p.causal ? (kv_len - n_new + q0 + tok_local) : (kv_len - 1), kv_hi - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + a * kBN;
    const uint32_t p_addr = tmem + lane_base + COL_P + a * (kBN / 2);
    const uint32_t o_addr = tmem + lane_base + COL_O;
    // the warp of the other group that owns the same rows publishes its reference on its barrier
    const uint32_t bar_mine = bar(B_MREF + 4 * a + (warp & 3)), bar_other = bar(B_MREF + 4 * (1 - a) + (warp & 3));
    const float sc = p.scale_log2;
    float m_mine = -INFINITY, l = 0.f;        // l is scaled to the reference m_mine
    bool ok = true;
    for (int j = a; j < n_blocks; j += 2) {
      if (!warp_wait(bar(B_SFULL + a), (j >> 1) & 1, p.status)) { ok = false; break; }
      tc_fence_after();
      const int t0 = j * kBN;
      uint32_t r[kBN];
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(bar(B_SFREE + a) + lead);  // S_a may take Q K^T of block j+2
      if (t0 + kBN - 1 > limit) {
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (t0 + i > limit) r[i] = 0xff800000u;  // -inf
      }
      float mx;
      {
        float m8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) m8[i] = __uint_as_float(r[i]);
#pragma unroll
        for (int i = 8; i + 15 < kBN; i += 16) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            m8[q] = fmax3(m8[q], __uint_as_float(r[i + 2 * q]), __uint_as_float(r[i + 2 * q + 1]));
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) m8[q] = fmaxf(m8[q], __uint_as_float(r[kBN - 8 + q]));  // 8 + 7 * 16 = 120 done
        mx = fmaxf(fmax3(m8[0], m8[1], m8[2]), fmaxf(fmax3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7])));
      }
      const float m_tile = mx * sc;
      // the reference maximum block j-1 left (the other group's latest), then ours
      float m_prev = -INFINITY;
      if (j > 0) {
        // block j-1 is the other group's ((j-1)/2)-th. In the same poll: P_a is free once P V of block
        // j-2 has read it (long ago, as a rule). Products finish in order, so the other group's pvdone
        // barrier is then past block j-3 and a wait for block j-1 on it cannot be answered by an older phase.
        const bool both = j >= 2;
        if (!warp_wait2(bar_other, ((j - 1) >> 1) & 1, both ? bar(B_PVDONE + a) : bar_other,
                        both ? ((j - 2) >> 1) & 1 : ((j - 1) >> 1) & 1, p.status)) {
          ok = false;
          break;
        }
        m_prev = mref[(1 - a) * 128 + row];
      }
      float m_new = m_prev;
      if (m_tile > m_prev + kRescaleThreshold || (m_prev == -INFINITY && m_tile > -INFINITY)) m_new = m_tile;
      if (j + 1 < n_blocks) {
        mref[a * 128 + row] = m_new;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_mine);
      }
      if (m_new != m_mine) {  // bring this group's partial sum to the current reference
        l *= (m_mine == -INFINITY) ? 0.f : exp2f(m_mine - m_new);
        m_mine = m_new;
      }
      if (j > 0 && __any_sync(0xffffffffu, m_new != m_prev)) {
        // O takes in block j-1 until that product has finished
        if (!warp_wait(bar(B_PVDONE + (1 - a)), ((j - 1) >> 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const float factor = (m_prev == -INFINITY) ? 0.f : exp2f(m_prev - m_new);
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st32(o_addr + c * 32, o);
        }
      }
      const float off = (m_new == -INFINITY) ? 0.f : m_new;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1, e0, e1;
          ffma2(x0, x1, __uint_as_float(r[c * 32 + 2 * i]), __uint_as_float(r[c * 32 + 2 * i + 1]), sc, sc, -off, -off);
          e0 = ex2(x0);
          e1 = ex2(x1);
          fadd2(ls[2 * (i & 1)], ls[2 * (i & 1) + 1], ls[2 * (i & 1)], ls[2 * (i & 1) + 1], e0, e1);
          pk[i] = pack2<T>(e0, e1);
        }
        tmem_st16(p_addr + c * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(bar(B_PFULL + a) + lead);
    }
    // ---- epilogue: both groups' partial sums at the final reference, each stores half of head_dim
    lsum[a * 128 + row] = l;
    mfin[a * 128 + row] = m_mine;
    named_sync(9, 256);
    // the last product: first this group's own last one (its barrier is at most one phase behind),
    // after which the other group's barrier is in the phase of the very last block
    const int j_last = n_blocks - 1 - ((n_blocks - 1 - a) & 1);
    if (ok && j_last >= 0) ok = warp_wait(bar(B_PVDONE + a), (j_last >> 1) & 1, p.status);
    if (ok) ok = warp_wait(bar(B_PVDONE + ((n_blocks - 1) & 1)), ((n_blocks - 1) >> 1) & 1, p.status);
    if (ok) {
      tc_fence_after();
      // O is scaled to the reference of the group that worked on the last block
      const int last = (n_blocks - 1) & 1;
      const float m_fin = mfin[last * 128 + row], m_oth = mfin[(1 - last) * 128 + row];
      const float l_oth = lsum[(1 - last) * 128 + row];
      const float l_all = lsum[last * 128 + row] + ((m_oth == -INFINITY) ? 0.f : l_oth * exp2f(m_oth - m_fin));
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + (int64_t)(q_begin + q0 + tok_local) * p.out_stride +
               (int64_t)(kv_head * G + head) * D + a * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + a * 64 + c * 32, o);
        tmem_wait_ld();
        if (row_live) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w[i] = pack2<T>(__uint_as_float(o[v * 8 + 2 * i]) * inv, __uint_as_float(o[v * 8 + 2 * i + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  // ---- teardown: both CTAs meet (the peer's shared memory and TMEM are in use until here) -------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
  }
}

// ---- host -------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

int ilog2_exact(int x) {
  if (x <= 0 || (x & (x - 1)) != 0) return -1;
  int l = 0;
  while ((1 << l) < x) ++l;
  return l;
}

}  // namespace
}  // namespace dsv

extern "C" {

int dsv_prefill_plan(const int32_t* qo_indptr_host, const int32_t* kv_len_host, int batch, int n_q_heads,
                     int n_kv_heads, int head_dim, int page_size, int dtype, int causal, int min_new_tokens,
                     int32_t* plan_host, int64_t plan_capacity_i32, int64_t* plan_used_i32) {
  using namespace dsv;
  DSV_REQUIRE(qo_indptr_host && kv_len_host && plan_host && plan_used_i32, "prefill_plan: null pointer argument");
  DSV_REQUIRE(batch >= 0, "prefill_plan: negative batch");
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "prefill_plan: bad head counts");
  const int G = n_q_heads / n_kv_heads;
  DSV_REQUIRE(G <= 128 && 128 % G == 0, "prefill_plan: GQA group %d must divide 128", G);
  const int tq = 128 / G;
  struct Item { int req, q0, nq, hi; };
  // A pair item is two q tiles of one request for a cluster of two CTAs (one tile each); a request's
  // last tile, when it is alone, is a single-CTA item. The pair kernel exists for head_dim 128;
  // without it an item is two q tiles for one CTA.
  std::vector<Item> items, pairs;
  // (the pair kernel is still the slower one on the benchmark shape: opt-in until it is not)
  const char* pairs_env = std::getenv("DESERVE_PREFILL_PAIRS");
  const bool use_pairs = head_dim == 128 && page_size >= 16 && pairs_env != nullptr && pairs_env[0] == '1';
  for (int i = 0; i < batch; ++i) {
    const int n = qo_indptr_host[i + 1] - qo_indptr_host[i];
    const int len = kv_len_host[i];
    DSV_REQUIRE(n >= 0 && len >= n, "prefill_plan: request %d has %d new tokens but kv length %d", i, n, len);
    if (n < min_new_tokens) continue;  // left to another kernel (decode rows of a mixed batch)
    int q0 = 0;
    while (q0 < n) {
      const int left = n - q0;
      const bool pair = use_pairs && left > tq;
      const int nq = std::min(2 * tq, left);
      const int hi = causal ? len - n + q0 + nq : len;  // kv positions the item's last token sees
      (pair ? pairs : items).push_back({i, q0, nq, hi});
      q0 += nq;
    }
  }
  const int64_t need = kPlanHeader + 4 * (int64_t)(items.size() + pairs.size());
  *plan_used_i32 = need;
  if (need > plan_capacity_i32)
    return fail(DSV_E_WORKSPACE, "prefill_plan: plan needs %lld int32, capacity %lld", (long long)need,
                (long long)plan_capacity_i32);
  // Most work first, but a request's items stay together: they read the same K/V and then find it in
  // L2. Requests by their longest item, inside a request the longest item first.
  std::vector<int> req_hi(batch, 0);
  for (const Item& it : items) req_hi[it.req] = std::max(req_hi[it.req], it.hi);
  for (const Item& it : pairs) req_hi[it.req] = std::max(req_hi[it.req], it.hi);
  auto longest_first = [&](const Item& a, const Item& b) {
    if (a.req != b.req) return req_hi[a.req] != req_hi[b.req] ? req_hi[a.req] > req_hi[b.req] : a.req < b.req;
    return a.hi > b.hi;
  };
  std::stable_sort(items.begin(), items.end(), longest_first);
  std::stable_sort(pairs.begin(), pairs.end(), longest_first);
  plan_host[0] = kPrefillMagic;
  plan_host[1] = (int32_t)items.size();
  plan_host[2] = tq;
  plan_host[3] = causal ? 1 : 0;
  plan_host[4] = batch;
  plan_host[5] = kPlanHeader;
  plan_host[6] = n_q_heads;
  plan_host[7] = n_kv_heads;
  plan_host[8] = (int32_t)pairs.size();
  plan_host[9] = kPlanHeader + 4 * (int32_t)items.size();
  plan_host[10] = plan_host[11] = 0;
  for (size_t k = 0; k < items.size() + pairs.size(); ++k) {
    const Item& src = k < items.size() ? items[k] : pairs[k - items.size()];
    int32_t* it = plan_host + kPlanHeader + 4 * k;
    it[0] = src.req; it[1] = src.q0; it[2] = src.nq; it[3] = src.hi;
  }
  (void)dtype;
  return DSV_OK;
}

int dsv_paged_prefill(const void* q, int64_t q_stride_tok, const int32_t* qo_indptr, const void* pages_layer,
                      int64_t page_stride, int64_t num_pages, const int32_t* kv_indices, const int32_t* kv_indptr,
                      const int32_t* kv_last_page_len, void* out, int64_t out_stride_tok, const int32_t* plan_host,
                      const int32_t* plan_dev, int batch, int nnz, int n_q_heads, int n_kv_heads, int head_dim,
                      int page_size, int dtype, float sm_scale, int causal, void* stream) {
  using namespace dsv;
  DSV_REQUIRE(dtype_ok(dtype), "prefill: unknown dtype %d", dtype);
  DSV_REQUIRE(batch >= 0 && nnz >= 0, "prefill: negative batch or nnz");
  if (batch == 0 || nnz == 0) return DSV_OK;
  DSV_REQUIRE(q && qo_indptr && pages_layer && kv_indices && kv_indptr && kv_last_page_len && out && plan_host && plan_dev,
              "prefill: null pointer argument");
  if (dtype == DSV_F32)
    return fail(DSV_E_UNSUPPORTED, "prefill: fp32 K/V has no tensor-core kernel here (fp16 and bf16 only)");
  DSV_REQUIRE(n_q_heads > 0 && n_kv_heads > 0 && n_q_heads % n_kv_heads == 0, "prefill: bad head counts");
  const int G = n_q_heads / n_kv_heads;
  DSV_REQUIRE(G <= 128 && 128 % G == 0, "prefill: GQA group %d must divide 128", G);
  DSV_REQUIRE(head_dim == 64 || head_dim == 128, "prefill: head_dim %d not in {64,128}", head_dim);
  const int ps_log2 = ilog2_exact(page_size);
  DSV_REQUIRE(ps_log2 >= 0, "prefill: page_size %d must be a power of two", page_size);
  DSV_REQUIRE(num_pages > 0 && num_pages < (1ll << 30), "prefill: num_pages out of range");
  DSV_REQUIRE(plan_host[0] == kPrefillMagic && plan_host[4] == batch && plan_host[6] == n_q_heads &&
                  plan_host[7] == n_kv_heads && plan_host[3] == (causal ? 1 : 0),
              "prefill: plan does not belong to this call");
  DSV_REQUIRE(page_stride == (int64_t)2 * page_size * n_kv_heads * head_dim, "prefill: the page pool must be dense");
  DSV_REQUIRE(aligned16(q) && aligned16(pages_layer) && aligned16(out) && (q_stride_tok * 2) % 16 == 0 &&
                  (out_stride_tok * 2) % 16 == 0,
              "prefill: pointers and strides must be 16-byte aligned");
  DSV_REQUIRE(q_stride_tok >= (int64_t)n_q_heads * head_dim && out_stride_tok >= (int64_t)n_q_heads * head_dim,
              "prefill: token stride smaller than a row");
  const int n_items = plan_host[1], n_pairs = plan_host[8];
  DSV_REQUIRE(n_items >= 0 && n_pairs >= 0 && (n_pairs == 0 || (head_dim == 128 && page_size >= 16)), "prefill: corrupt plan");
  if (n_items == 0 && n_pairs == 0) return DSV_OK;
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return fail(DSV_E_CUDA, "prefill: cuTensorMapEncodeTiled is not available");
  const CUtensorMapDataType dt = dtype == DSV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUtensorMap q_map, kv_map, k_map, v_map;
  const bool merged = head_dim == 128 && page_size >= 16;  // 4 KB boxes: both halves of head_dim per 16 tokens
  {  // q: (64 elements, head, 64-element half, token); box = (64, G, 1, 128/G) -> rows token*G + head
    const cuuint64_t dims[4] = {64, (cuuint64_t)n_q_heads, (cuuint64_t)(head_dim / 64), (cuuint64_t)nnz};
    const cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, 128, (cuuint64_t)q_stride_tok * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)(128 / G)};
    if (enc(&q_map, dt, 4, const_cast<void*>(q), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fail(DSV_E_CUDA, "prefill: tensor map of q rejected");
  }
  {  // pages: (64 elements, token in page, head, 64-element half, 2*page + {K,V}); box = 16 tokens of one head and half
    const int bt = page_size < 16 ? page_size : 16;
    const cuuint64_t half_stride = (cuuint64_t)page_size * n_kv_heads * head_dim * 2;
    const cuuint64_t dims[5] = {64, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, (cuuint64_t)(head_dim / 64),
                                (cuuint64_t)(2 * num_pages)};
    const cuuint64_t strides[4] = {(cuuint64_t)n_kv_heads * head_dim * 2, (cuuint64_t)head_dim * 2, 128, half_stride};
    const cuuint32_t box[5] = {64, (cuuint32_t)bt, 1, 1, 1};
    if (enc(&kv_map, dt, 5, const_cast<void*>(pages_layer), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fail(DSV_E_CUDA, "prefill: tensor map of the pages rejected");
  }
  k_map = kv_map;
  v_map = kv_map;
  if (merged) {
    // K boxes of 16 tokens x both halves of head_dim in one 4 KB box. The token index is
    // split in (token mod 8, token / 8) with the half of head_dim between them, so that the box lands as
    // [8-token group][half][8 tokens][128 B]: 8-token groups 2 KB apart for either half, which one MMA
    // descriptor can walk. Dimensions: element, token mod 8, head * 2 + half, token / 8 in the page, 2 * page + {K, V}.
    const cuuint64_t half_stride = (cuuint64_t)page_size * n_kv_heads * head_dim * 2;
    const cuuint64_t dims[5] = {64, 8, (cuuint64_t)(2 * n_kv_heads), (cuuint64_t)(page_size / 8), (cuuint64_t)(2 * num_pages)};
    const cuuint64_t strides[4] = {(cuuint64_t)n_kv_heads * head_dim * 2, 128, (cuuint64_t)8 * n_kv_heads * head_dim * 2,
                                   half_stride};
    const cuuint32_t box[5] = {64, 8, 2, 2, 1};
    if (enc(&k_map, dt, 5, const_cast<void*>(pages_layer), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fail(DSV_E_CUDA, "prefill: tensor map of the K boxes rejected");
    // V boxes: the pages' own dimension order with both halves in the box -> [half][16 tokens][128 B]
    const cuuint64_t vdims[5] = {64, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, 2, (cuuint64_t)(2 * num_pages)};
    const cuuint64_t vstrides[4] = {(cuuint64_t)n_kv_heads * head_dim * 2, (cuuint64_t)head_dim * 2, 128, half_stride};
    const cuuint32_t vbox[5] = {64, 16, 1, 2, 1};
    if (enc(&v_map, dt, 5, const_cast<void*>(pages_layer), vdims, vstrides, vbox, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return fail(DSV_E_CUDA, "prefill: tensor map of the V boxes rejected");
  }
  PrefillParams p;
  p.qo_indptr = qo_indptr; p.kv_indices = kv_indices; p.kv_indptr = kv_indptr; p.kv_last_page_len = kv_last_page_len;
  p.out = out; p.items = reinterpret_cast<const int4*>(plan_dev + plan_host[5]);
  DSV_REQUIRE(aligned16(p.items), "prefill: device plan must be 16-byte aligned");
  p.out_stride = out_stride_tok; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.ps_log2 = ps_log2;
  p.num_pages = (int)num_pages; p.causal = causal ? 1 : 0; p.scale_log2 = sm_scale * kLog2e;
  p.status = device_status_ptr();
  auto go = [&](auto kernel, dim3 grid, int threads, size_t smem, const PrefillParams& pp) -> cudaError_t {
    cudaError_t er = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (er != cudaSuccess) return er;
    kernel<<<grid, threads, smem, (cudaStream_t)stream>>>(q_map, kv_map, k_map, v_map, pp);
    return cudaGetLastError();
  };
  cudaError_t e = cudaSuccess;
  if (n_pairs > 0) {  // the long items first: a cluster of two CTAs per item and kv head
    PrefillParams pp = p;
    pp.items = reinterpret_cast<const int4*>(plan_dev + plan_host[9]);
    const size_t smem = (size_t)128 * 128 * 2 + (size_t)kPKStages * (2 * 64 * 128) + (size_t)kPVStages * (kBN * 128) +
                        6 * 128 * 4 + 512 + 1024;
    const dim3 grid(2u * (unsigned)n_pairs * (unsigned)n_kv_heads);
    auto go_pair = [&](auto kernel) -> cudaError_t {
      cudaError_t er = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (er != cudaSuccess) return er;
      kernel<<<grid, kPairThreads, smem, (cudaStream_t)stream>>>(q_map, kv_map, k_map, pp);
      return cudaGetLastError();
    };
    e = dtype == DSV_BF16 ? go_pair(prefill_pair_kernel<__nv_bfloat16>) : go_pair(prefill_pair_kernel<__half>);
  }
  if (e == cudaSuccess && n_items > 0) {
    const size_t smem = (size_t)2 * 128 * head_dim * 2 + (size_t)(2 + kVStages) * kBN * head_dim * 2 + 256 + 1024;
    const dim3 grid((unsigned)n_items * (unsigned)n_kv_heads);
    if (dtype == DSV_BF16)
      e = merged ? go(prefill_kernel<__nv_bfloat16, 128, true>, grid, kThreads, smem, p)
                 : head_dim == 128 ? go(prefill_kernel<__nv_bfloat16, 128, false>, grid, kThreads, smem, p)
                                   : go(prefill_kernel<__nv_bfloat16, 64, false>, grid, kThreads, smem, p);
    else
      e = merged ? go(prefill_kernel<__half, 128, true>, grid, kThreads, smem, p)
                 : head_dim == 128 ? go(prefill_kernel<__half, 128, false>, grid, kThreads, smem, p)
                                   : go(prefill_kernel<__half, 64, false>, grid, kThreads, smem, p);
  }
  if (e != cudaSuccess) return fail(DSV_E_CUDA, "prefill launch failed: %s", cudaGetErrorString(e));
  return DSV_OK;
}

}  // extern "C"
