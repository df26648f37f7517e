// Prefill attention on the 5th-generation tensor cores: Q K^T and P V are tcgen05.mma instructions with the score tile S and
// the output tile O in tensor memory, K/V tiles arrive through the block table as TMA boxes, and four warps run the online
// softmax with one thread per query row (a TMEM lane), so row maxima and sums need no shuffles.
//
// Same semantics as paged_attention_kernel (attention.cu: packed variable-length queries over a block-table cache, GQA rows
// (token, head of the group) sharing one K/V stream, causal / sliding-window / bidirectional masks, sinks, soft-capping;
// reference ops: GroupQueryAttention / PagedAttention, src/python/py/models/builders/base.py:3315-3386, 3484-3536).  It serves
// the requests of a launch that have at least TCA_MIN_ROWS query rows; the other requests (decode rows, short verify rows) are
// left to the bandwidth-bound kernel, which skips the ones taken here.
//
// One CTA = (request, kv head, 128 query rows).  Roles:
//   warps 0-7  softmax: a row (TMEM lane) is shared by two threads, one per half of the tile's key columns (warp w serves the
//              lane quarter w % 4, which is the only one it may address, and column half w / 4).  Per K/V tile: read S from TMEM,
//              scale / soft-cap / mask, row maximum (the two halves meet through shared memory), exponentials, bf16 P written
//              over S in TMEM (the A operand of P V is read from tensor memory), rescale O in TMEM when the maximum moved.
//   warps 8,9  TMA producers of the K ring and of the V ring: per 16 keys and 64 dims one box (the cache as a 2-D tensor
//              [slots, kv_heads * head_dim], 128-byte swizzle); the lanes look their blocks up in parallel.
//   warp 10    MMA issuer (one lane): S[b] = Q K_j^T into one of three S buffers, two tiles ahead of the softmax warps;
//              O += P_j V_j with V as the MN-major B operand (keys are its K dimension) as soon as P_j is there.
// The softmax loop is plain (read S, mask, maximum, exchange, exponentials, P back into TMEM): a software-pipelined form
// (exponentials of tile j interleaved with the load and maximum of tile j + 1) measured slower, 457 against 591 TFLOP/s at 4096
// tokens, because its loop body outgrew the instruction cache and its extra waits cost more than the overlap gave.  The scale is
// folded into the exponent's multiply-add.  Registers move from the producer / issuer warps to the softmax warps (setmaxnreg).
// Row tiles are dispatched from the end of the prompt (most keys) to its start, so the grid's tail is short CTAs (591 -> 658).
//
// Every wait on an mbarrier is bounded (mbar_wait_bounded); a wait that runs out sets the CTA's abort flag and the device status
// word; the producers and the issuer leave their loops, the softmax warps keep walking theirs without waiting (they share a
// named barrier per warp pair, which has no time limit, so none of them may leave early), the producer waits (bounded) for
// copies in flight, TMEM is freed and the kernel returns.
// The cache must hold finite values in every slot of a block that is in use (PagedKVCache allocates zeros): keys past the end
// of a request inside its last 16-key group are masked (P = 0) but still multiplied.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace ogb {

bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);  // gemm_tcgen05.cu

constexpr int TCA_BM = 128;
constexpr int TCA_SOFTMAX_THREADS = 256;
constexpr int TCA_THREADS = TCA_SOFTMAX_THREADS + 128;      // warps 8..11: K producer, V producer, MMA issuer, one spare
constexpr int TCA_K_WARP = 8, TCA_V_WARP = 9, TCA_MMA_WARP = 10;
constexpr int TCA_REGS_SOFTMAX = 224, TCA_REGS_OTHER = 40;   // after setmaxnreg: 256 x 224 + 128 x 40 registers
constexpr float TCA_LOG2E = 1.4426950408889634f;
constexpr float TCA_RESCALE_GAP = 8.f;   // log2 units

struct TcAttnParams {
  const __nv_bfloat16* q; int q_stride;
  const int32_t* cu_seqlens; const int32_t* past_lens;
  const int32_t* block_table; int table_cols; int block_size;
  __nv_bfloat16* out; int out_stride;
  const float* sinks;
  float scale, softcap;
  int window, B, Hq, Hkv, min_rows;
  int* status;
};

template <int D, int BN>
struct TcaCfg {
  static constexpr int HALVES = D / 64;
  static constexpr int Q_BYTES = TCA_BM * D * 2;
  static constexpr int KV_TILE = BN * D * 2;                 // one K (or V) tile
  // K and V tiles have rings of their own: a K tile is free as soon as its Q K^T is done (one tile period earlier than the
  // V tile of the same keys), and the loads must run two to three tile periods ahead of their use to hide their latency.
  static constexpr int BUDGET = 227 * 1024 - 1024 - 1536 - Q_BYTES;      // 1 KiB of alignment slack, static shared memory
  static constexpr int RING = BUDGET / KV_TILE >= 8 ? 8 : BUDGET / KV_TILE;
  static constexpr int K_STAGES = (RING + 1) / 2, V_STAGES = RING / 2;
  static constexpr int SMEM = 1024 + Q_BYTES + (K_STAGES + V_STAGES) * KV_TILE;
  static constexpr int S_BUFS = 3;
  static constexpr int S_COLS = BN, O_COL = S_BUFS * BN;
  static constexpr int COLS_USED = S_BUFS * BN + D;
  static constexpr int TMEM_COLS = COLS_USED <= 128 ? 128 : (COLS_USED <= 256 ? 256 : 512);
  static constexpr int CTAS_PER_SM = 1;
};

// MN-major operand with the 128-byte swizzle: 64 contiguous elements per 128-byte row, rows are K indices; 8-row groups along
// K are `sbo` bytes apart, 64-element groups along MN are `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]: A is 128 lanes x K values, two 16-bit values per 32-bit column.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int D, int BN>
__global__ void __launch_bounds__(TCA_THREADS, TcaCfg<D, BN>::CTAS_PER_SM)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, TcAttnParams p) {
  using Cfg = TcaCfg<D, BN>;
  constexpr int HALVES = Cfg::HALVES, KS = Cfg::K_STAGES, VS = Cfg::V_STAGES;
  extern __shared__ __align__(128) uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [HALVES][128 rows][128 B]
  uint8_t* sK = sQ + Cfg::Q_BYTES;                     // [KS][HALVES][BN keys][128 B]
  uint8_t* sV = sK + KS * Cfg::KV_TILE;                // [VS][HALVES][BN keys][128 B]
  __shared__ uint64_t k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[Cfg::S_BUFS], p_full[Cfg::S_BUFS], o_done[Cfg::S_BUFS], q_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  // Row maxima of the two column halves, [tile parity][half][row] as bf16 (rounded up: a reference maximum only has to be
  // the same on both sides and not below the true one); at the end the same bytes carry the halves' sums as [half][row] fp32.
  __shared__ __align__(16) __nv_bfloat16 xchg[2][2][TCA_BM];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int tok0 = p.cu_seqlens[b];
  const int q_len = p.cu_seqlens[b + 1] - tok0;
  const int rows = q_len * G;
  // CTAs are dispatched in block-index order: the last row tiles of a causal prompt see the most keys, so they go first and
  // the tail of the grid is made of short CTAs
  const int row0 = int(gridDim.x - 1 - blockIdx.x) * TCA_BM;
  if (rows < p.min_rows || row0 >= rows) return;      // before anything is allocated
  const int past = p.past_lens[b];
  const bool full = p.window < 0;
  const int32_t* table = p.block_table + size_t(b) * p.table_cols;
  const int last_tq = min(q_len - 1, (row0 + TCA_BM - 1) / G);
  const int kv_hi = full ? past : past + last_tq + 1;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, past + row0 / G - p.window + 1);
  const int tile_begin = kv_lo / BN;
  const int n_tiles = kv_hi > kv_lo ? (kv_hi + BN - 1) / BN - tile_begin : 0;

  if (tid == 0) {
    for (int i = 0; i < KS; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < VS; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < Cfg::S_BUFS; ++i) mbar_init(&s_full[i], 1);
    for (int i = 0; i < Cfg::S_BUFS; ++i) { mbar_init(&p_full[i], TCA_SOFTMAX_THREADS); mbar_init(&o_done[i], 1); }
    mbar_init(&q_full, TCA_SOFTMAX_THREADS);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == TCA_K_WARP) {
    tmem_alloc(&tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_launch_dependents();        // only now: a dependent grid that also wants tensor memory starts after this CTA owns its share
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_p = &abort_flag;
  auto fail = [&](int code) {
    *abort_p = 1;
    if (p.status) atomicMax(p.status, code);
  };

  if (warp >= TCA_K_WARP) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TCA_REGS_OTHER));
  if (warp == TCA_K_WARP || warp == TCA_V_WARP) {
    // ------------------------------------------------------------------------------ TMA producers (K ring, V ring)
    const bool is_k = warp == TCA_K_WARP;
    const CUtensorMap* tmap = is_k ? &tmap_k : &tmap_v;
    uint64_t* full = is_k ? k_full : v_full;
    uint64_t* empty = is_k ? k_empty : v_empty;
    uint8_t* ring = is_k ? sK : sV;
    const int NS = is_k ? KS : VS;
    if (lane == 0) tma_prefetch_desc(tmap);
    const int last_group = max(0, (kv_hi - 1) / 16 * 16);
    int issued = 0;
    for (int it = 0; it < n_tiles; ++it) {
      const int st = it % NS;
      if (it >= NS && !mbar_wait_bounded(&empty[st], ((it / NS) - 1) & 1, abort_p)) { if (lane == 0) fail(OGB_ERR_WAIT_TMA); break; }
      if (lane == 0) mbar_expect_tx(&full[st], Cfg::KV_TILE);
      __syncwarp();
      // Key groups past the end of the range re-read the last valid group (their scores are masked), so every stage
      // receives the same byte count.
      if (lane < BN / 16) {
        const int j0 = min((tile_begin + it) * BN + lane * 16, last_group);
        const int slot0 = table[j0 / p.block_size] * p.block_size + j0 % p.block_size;
        uint8_t* dst = ring + st * Cfg::KV_TILE + lane * 16 * 128;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * (BN * 128), tmap, &full[st], kvh * D + h * 64, slot0);
      }
      issued = it + 1;
    }
    if (*abort_p) {
      // copies in flight must land before the shared memory goes away
      for (int it = max(0, issued - NS); it < issued; ++it) {
        int dummy = 0;
        mbar_wait_bounded(&full[it % NS], (it / NS) & 1, &dummy, 20000000ull);
      }
    }
  } else if (warp == TCA_MMA_WARP) {
    // ------------------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = umma_idesc_f16(TCA_BM, BN, 1);
    constexpr uint32_t idesc_pv = umma_idesc_f16(TCA_BM, D, 1) | (1u << 16);     // B operand MN-major
    const uint32_t q_addr = smem_u32(sQ), k_ring = smem_u32(sK), v_ring = smem_u32(sV);
    constexpr uint32_t lbo = BN * 128, sbo = 1024;       // between the 64-dim halves of V; between 8-key groups
    bool ok = mbar_wait_bounded(&q_full, 0, abort_p);
    if (!ok && lane == 0) fail(OGB_ERR_WAIT_MMA);
    auto issue_qk = [&](int it) -> bool {
      const int st = it % KS;
      if (!mbar_wait_bounded(&k_full[st], (it / KS) & 1, abort_p)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = k_ring + st * Cfg::KV_TILE;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t da = umma_desc_sw128(q_addr + (ks >> 2) * (TCA_BM * 128) + (ks & 3) * 32);
          const uint64_t db = umma_desc_sw128(k_addr + (ks >> 2) * (BN * 128) + (ks & 3) * 32);
          umma_f16(tmem_base + (it % Cfg::S_BUFS) * Cfg::S_COLS, da, db, idesc_qk, ks > 0);
        }
        umma_commit(&s_full[it % Cfg::S_BUFS]);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
      return true;
    };
    // Q K^T runs three tiles ahead (three S buffers; P_j replaces S_j in place and the buffer is free again after P_j V_j,
    // which the in-order tensor pipe finishes before the Q K^T issued behind it starts)
    for (int it = 0; ok && it < min(Cfg::S_BUFS, n_tiles); ++it) ok = issue_qk(it);
    if (!ok && lane == 0) fail(OGB_ERR_WAIT_TMA);
    for (int it = 0; ok && it < n_tiles; ++it) {
      // (barriers per S buffer: a waiter can then never be two phases behind, whichever side runs ahead)
      if (!mbar_wait_bounded(&p_full[it % Cfg::S_BUFS], (it / Cfg::S_BUFS) & 1, abort_p)) { if (lane == 0) fail(OGB_ERR_WAIT_MMA); ok = false; break; }
      const int st = it % VS;
      if (!mbar_wait_bounded(&v_full[st], (it / VS) & 1, abort_p)) { if (lane == 0) fail(OGB_ERR_WAIT_TMA); ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = v_ring + st * Cfg::KV_TILE;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint64_t db = umma_desc_sw128_mn(v_addr + ks * 16 * 128, lbo, sbo);
          umma_f16_ta(tmem_base + Cfg::O_COL, tmem_base + (it % Cfg::S_BUFS) * Cfg::S_COLS + ks * 8, db, idesc_pv, (it > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&o_done[it % Cfg::S_BUFS]);
      }
      __syncwarp();
      if (it + Cfg::S_BUFS < n_tiles && !issue_qk(it + Cfg::S_BUFS)) { if (lane == 0) fail(OGB_ERR_WAIT_TMA); ok = false; break; }
    }
  }
  // (warp 11 is the spare of the fourth warpgroup: register reallocation works on whole warpgroups)
  } else {
    // ------------------------------------------------------------------------------ softmax warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TCA_REGS_SOFTMAX));
    constexpr int HC = BN / 2;                 // key columns per thread and tile
    constexpr int OC = D / 2;                  // output columns per thread
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;
    const int gr = row0 + r;
    const bool valid = gr < rows;
    const int tq = valid ? gr / G : q_len - 1;
    const int hq = kvh * G + (valid ? gr % G : 0);
    const int qpos = past + tq;
    // The two warps of a lane quarter meet on a named barrier.  It has no time limit, so no softmax warp ever leaves the tile loop
    // early: after a bounded wait gave up (abort flag set) a warp keeps walking the loop - its waits then return at once - and
    // still arrives at every barrier its partner arrives at.
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory"); };
    {
      const __nv_bfloat16* src = p.q + size_t(tok0 + tq) * p.q_stride + size_t(hq) * D;
#pragma unroll
      for (int cc = 0; cc < D / 16; ++cc) {
        const int c = half * (D / 16) + cc;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
        *reinterpret_cast<uint4*>(sQ + (c >> 3) * (TCA_BM * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(&q_full);
    }
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
    const bool capped = p.softcap > 0.f;
    const float kmul = capped ? 1.f : p.scale * TCA_LOG2E;        // exponent = s * kmul - reference maximum
    const float inv_cap = capped ? p.scale / p.softcap : 0.f, capl = p.softcap * TCA_LOG2E;
    // a tile every key of which every row of this lane quarter sees needs no masks
    const int wq_lo = past + min(q_len - 1, (row0 + quarter * 32) / G), wq_hi = past + min(q_len - 1, (row0 + quarter * 32 + 31) / G);
    const bool rows_full = row0 + quarter * 32 + 31 < rows;
    auto tile_interior = [&](int it) {
      const int j0 = (tile_begin + it) * BN;
      return j0 >= kv_lo && j0 + BN <= kv_hi && (full || j0 + BN - 1 <= wq_lo) && (p.window <= 0 || j0 > wq_hi - p.window) && rows_full;
    };
    auto issue_loads = [&](int it, float (&dst)[HC]) {
#pragma unroll
      for (int c = 0; c < HC / 16; ++c) {
        uint32_t v[16];
        tmem_ld16(lane_base + (it % Cfg::S_BUFS) * Cfg::S_COLS + half * HC + c * 16, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) dst[c * 16 + e] = __uint_as_float(v[e]);
      }
    };
    // soft-cap / mask 16 scores of tile `it` in place and return their maximum (raw units: times kmul gives the exponent)
    auto prep16 = [&](int it, float (&x)[HC], int c, bool interior) -> float {
      if (capped) {
#pragma unroll
        for (int e = 0; e < 16; ++e) x[c * 16 + e] = capl * tanhf(x[c * 16 + e] * inv_cap);
      }
      if (!interior) {
        const int jb = (tile_begin + it) * BN + half * HC + c * 16;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int j = jb + e;
          bool vis = valid && j >= kv_lo && j < kv_hi && (full || j <= qpos);
          if (p.window > 0) vis = vis && j > qpos - p.window;
          x[c * 16 + e] = vis ? x[c * 16 + e] : -INFINITY;
        }
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 16; e += 4) {
        m4[0] = fmaxf(m4[0], x[c * 16 + e]); m4[1] = fmaxf(m4[1], x[c * 16 + e + 1]);
        m4[2] = fmaxf(m4[2], x[c * 16 + e + 2]); m4[3] = fmaxf(m4[3], x[c * 16 + e + 3]);
      }
      return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
    };
    // row maximum of a tile from this half's maximum: meet the partner half through shared memory
    auto exchange_max = [&](int it, float mx_raw) -> float {
      const __nv_bfloat16 mxb = __float2bfloat16_ru(mx_raw * kmul);
      xchg[it & 1][half][r] = mxb;
      pair_sync();
      return fmaxf(__bfloat162float(mxb), __bfloat162float(xchg[it & 1][half ^ 1][r]));
    };
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
      if (ok && !mbar_wait_bounded(&s_full[it % Cfg::S_BUFS], (it / Cfg::S_BUFS) & 1, abort_p)) { fail(OGB_ERR_WAIT_MMA); ok = false; }
      tc_fence_after();
      float sc[HC];
      issue_loads(it, sc);
      tmem_ld_wait();
      const bool interior = tile_interior(it);
      float mx_raw = -INFINITY;
#pragma unroll
      for (int c = 0; c < HC / 16; ++c) mx_raw = fmaxf(mx_raw, prep16(it, sc, c, interior));
      const float mx_cur = exchange_max(it, mx_raw);
      // lazy maximum: move the reference only when the row maximum outgrew it by more than the gap (both halves decide alike)
      float alpha = 1.f;
      bool moved = false;
      if (mx_cur > m_ref + TCA_RESCALE_GAP || (m_ref == -INFINITY && mx_cur > -INFINITY)) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx_cur);
        m_ref = mx_cur;
        moved = true;
      }
      const float nms = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[HC / 2];
#pragma unroll
      for (int e = 0; e < HC; e += 4) {
        const float p0 = exp2f(fmaf(sc[e], kmul, nms)), p1 = exp2f(fmaf(sc[e + 1], kmul, nms));
        const float p2 = exp2f(fmaf(sc[e + 2], kmul, nms)), p3 = exp2f(fmaf(sc[e + 3], kmul, nms));
        sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
        pk[e / 2] = pack_bf16x2(p0, p1);
        pk[e / 2 + 1] = pack_bf16x2(p2, p3);
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      if (it > 0 && __any_sync(0xffffffffu, moved)) {
        if (ok && !mbar_wait_bounded(&o_done[(it - 1) % Cfg::S_BUFS], ((it - 1) / Cfg::S_BUFS) & 1, abort_p)) { fail(OGB_ERR_WAIT_MMA); ok = false; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < OC / 16; ++c) {
          uint32_t v[16];
          tmem_ld16(lane_base + Cfg::O_COL + half * OC + c * 16, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
          tmem_st16(lane_base + Cfg::O_COL + half * OC + c * 16, v);
        }
      }
      // P replaces S in place: two bf16 values per 32-bit column, this half's keys in columns [half * HC / 2, +HC / 2)
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) {
        uint32_t v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = pk[c * 16 + e];
        tmem_st16(lane_base + (it % Cfg::S_BUFS) * Cfg::S_COLS + half * (HC / 2) + c * 16, v);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[it % Cfg::S_BUFS]);
    }
    ok = ok && !*abort_p;
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done[(n_tiles - 1) % Cfg::S_BUFS], ((n_tiles - 1) / Cfg::S_BUFS) & 1, abort_p)) { fail(OGB_ERR_WAIT_MMA); ok = false; }
    tc_fence_after();
    // the row's sum is the two halves' sums (same reference maximum on both sides)
    pair_sync();                                                // the partner is done reading the last tile's maxima
    float* lsum = reinterpret_cast<float*>(&xchg[0][0][0]);     // [half][row]
    lsum[half * TCA_BM + r] = l;
    pair_sync();
    l += lsum[(half ^ 1) * TCA_BM + r];
    if (ok && !*abort_p) {
      float scale_o = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[hq] * TCA_LOG2E;
        const float mm = fmaxf(m_ref, sk);
        scale_o = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mm);
        l = l * scale_o + exp2f(sk - mm);
      }
      const float inv = l > 0.f ? scale_o / l : 0.f;
      __nv_bfloat16* po = p.out + size_t(tok0 + tq) * p.out_stride + size_t(hq) * D + half * OC;
#pragma unroll
      for (int c = 0; c < OC / 16; ++c) {
        uint32_t v[16];
        if (n_tiles > 0) {
          tmem_ld16(lane_base + Cfg::O_COL + half * OC + c * 16, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = 0u;
        }
        if (valid) {
          uint4 lo, hi;
          lo.x = pack_bf16x2(__uint_as_float(v[0]) * inv, __uint_as_float(v[1]) * inv);
          lo.y = pack_bf16x2(__uint_as_float(v[2]) * inv, __uint_as_float(v[3]) * inv);
          lo.z = pack_bf16x2(__uint_as_float(v[4]) * inv, __uint_as_float(v[5]) * inv);
          lo.w = pack_bf16x2(__uint_as_float(v[6]) * inv, __uint_as_float(v[7]) * inv);
          hi.x = pack_bf16x2(__uint_as_float(v[8]) * inv, __uint_as_float(v[9]) * inv);
          hi.y = pack_bf16x2(__uint_as_float(v[10]) * inv, __uint_as_float(v[11]) * inv);
          hi.z = pack_bf16x2(__uint_as_float(v[12]) * inv, __uint_as_float(v[13]) * inv);
          hi.w = pack_bf16x2(__uint_as_float(v[14]) * inv, __uint_as_float(v[15]) * inv);
          *reinterpret_cast<uint4*>(po + c * 16) = lo;
          *reinterpret_cast<uint4*>(po + c * 16 + 8) = hi;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == TCA_K_WARP) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int D, int BN>
static int LaunchTc(const TcAttnParams& p, const void* k_cache, const void* v_cache, int max_q_len, int cache_slots, cudaStream_t stream) {
  using Cfg = TcaCfg<D, BN>;
  auto kern = attention_tc_kernel<D, BN>;
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(kern, Cfg::SMEM, configured)) return -3;
  CUtensorMap mk, mv;
  memset(&mk, 0, sizeof(mk));
  memset(&mv, 0, sizeof(mv));
  if (!MakeMapBf16(&mk, k_cache, cache_slots, p.Hkv * D, p.Hkv * D, 16)) return -2;
  if (!MakeMapBf16(&mv, v_cache, cache_slots, p.Hkv * D, p.Hkv * D, 16)) return -2;
  const int G = p.Hq / p.Hkv;
  dim3 grid((max_q_len * G + TCA_BM - 1) / TCA_BM, p.Hkv, p.B);
  launch_pdl(kern, grid, dim3(TCA_THREADS), Cfg::SMEM, stream, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ogb

using namespace ogb;

// 1 when the tensor-core prefill kernel can serve this configuration (the caller then launches both kernels: this one takes the
// requests with at least `min_rows` query rows, ogb_paged_attention with skip_rows = min_rows the others).
OGB_API int ogb_attention_tc_supported(int D, int block_size, int kv_bits, int cache_slots) {
  return (D == 64 || D == 128) && block_size % 16 == 0 && kv_bits == 16 && cache_slots >= 16;
}

OGB_API int ogb_attention_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                             const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out, int out_stride,
                             const float* sinks, float scale, float softcap, int window, int B, int max_q_len, int Hq, int Hkv, int D,
                             int min_rows, int cache_slots, int* status, void* stream_) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (!ogb_attention_tc_supported(D, block_size, 16, cache_slots)) return -5;
  if (Hkv <= 0 || Hq % Hkv || (q_stride % 8) || (out_stride % 8)) return -1;
  if (((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) return -1;
  TcAttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride = q_stride;
  p.cu_seqlens = cu_seqlens; p.past_lens = past_lens; p.block_table = block_table; p.table_cols = table_cols; p.block_size = block_size;
  p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.sinks = sinks; p.scale = scale; p.softcap = softcap; p.window = window;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.min_rows = min_rows; p.status = status;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // 128 keys per tile (measured on B200 against 64: 457 vs 429 TFLOP/s at 4096 tokens, head_dim 128)
  if (D == 128) return LaunchTc<128, 128>(p, k_cache, v_cache, max_q_len, cache_slots, stream);
  return LaunchTc<64, 128>(p, k_cache, v_cache, max_q_len, cache_slots, stream);
}
