// Grouped expert GEMM over MXFP4 weights kept packed in HBM (QMoE semantics) on the 5th-generation tensor cores:
//     C[row, :] = A[row, :] * dequant(W[expert(row)])^T  (+ bias[expert]) (+ paired activation)
//
// Checkpoint semantics (reference: src/python/py/models/builders/base.py:4276-4408, builders/gptoss.py:653-847):
// FP4 e2m1 codes (sign, two exponent bits, one mantissa bit: 0, 0.5, 1, 1.5, 2, 3, 4, 6) with one power-of-two e8m0
// scale 2^(code - 127) per block of 32 along K.  The QMoE layout ([E, K, N/2] bytes + [E, N, K/32] scale codes) is
// repacked once at load time (ops/fp4.py) into tiles that one bulk copy streams: for every (expert, k-block of 64,
// tile of 128 output rows) a contiguous 4352-byte record
//     [128 rows][32 bytes of nibbles]  +  [128 rows][2 multiplier bytes]
// with the nibbles of each 32-bit word ordered so that `(word >> 4j)` puts two consecutive k values in the low
// nibbles of the two halves of a register.  HBM traffic is 4.25 bits per weight instead of 16.
//
// Expansion to bf16 without a table: the three magnitude bits of a code, placed at bits 8..6 of a bf16, are the
// number e2m1 * 2^-126 (the codes 0 and 1 land on zero and on the subnormal 2^-127, exactly as e2m1's own
// subnormal), so one bf16x2 multiply by 2^126 * 2^(scale - 127) = 2^(scale - 1) yields the weight exactly
// (PTX `mul.bf16x2` keeps subnormal inputs).  The multiplier byte stored in the record is that power's bf16
// exponent field, scale + 126; scale codes above 128 cannot be represented and are refused by the packer.
//
// fp16 form (the default when every block scale lies in 2^-14 .. 2^13): the tensor cores run fp16 x fp16 with the
// activations converted to fp16 by the row gather (and by the gate/up epilogue for the down projection).  A record word
// holds eight consecutive k values, byte i = (element i, element 4 + i); the eight words of a row's 64 k values are stored
// in the order (q, b) -> word 2q + b = k values 32b + 8q .. + 8, so that the 16 codes one lane of the streaming kernel
// below needs are 8 contiguous bytes.  `cvt.rn.f16x2.e2m1x2` expands a byte, `mul.f16x2` applies the block scale; the
// multiplier byte is scale code + 6 (the kernels subtract 118 to reach the fp16 exponent field of 2^(scale - 127)).
//
// Pipeline and epilogue are those of the int4 kernel (gemm_w4.cu): warp 0 streams records through a deep ring and the
// activation tiles through a ring of their own (4 or 8 deep), warps 2..9 expand a record into the swizzled K-major tile,
// warp 1 issues tcgen05.mma into tensor memory, warps 2..5 run the epilogue; two CTAs per SM.  The tile list of
// ogb_moe_sort selects the expert, first row and row count of each token tile.  Every wait is bounded.
//
// Where the time goes (clock64 trace of one CTA, 16-token tiles): a k-block takes about 1100 cycles per CTA, of which the
// MMA issuer spends about 500 between seeing its operands and having issued four tcgen05.mma (128 weight rows x 16 tokens
// x 16) and their commits; with two CTAs per SM that is one instruction per ~137 cycles, and a record of 4352 bytes would
// have to be consumed every 190 cycles to keep up with HBM.  More expander warps, more expanded tiles in flight, a deeper
// activation ring, tensor-map loads and four independent accumulators each left the time within 8 %.  The kernel
// therefore streams its weights at about 0.33 of the HBM rate (1.25x faster than the bf16 experts, which move 3.8x the
// bytes at the full rate).  It serves the larger token tiles (prompts); the 16-token tiles of decode steps go to the
// streaming kernel further down, which keeps the expanded weights in registers.
#include <cstdlib>

#include <cuda_fp16.h>

#include "gemm_common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int FP4_RECORD_BYTES = GEMM_BLOCK_N * 32 + GEMM_BLOCK_N * 2;  // 4352
constexpr int FP4_THREADS = 320;   // warp 0 producer, warp 1 MMA issuer, warps 2..9 expanders (2..5 also run the epilogue)
constexpr int FP4_DEQ_WARPS = 8;

template <int BT, int FP4_WBUF>
struct Fp4Cfg {
  static constexpr int A_TILE_BYTES = BT * GEMM_BLOCK_K * 2;
  static constexpr bool TWO_PER_SM = BT <= 64;
  static constexpr int BUDGET = TWO_PER_SM ? 100 * 1024 : 196 * 1024;
  // Activation tiles have their own, deeper ring: a tile is requested when the MMA that read the slot has finished, and
  // the copy takes most of a microsecond to arrive, so with two slots every k-block waited half that latency (the
  // kernel then ran at 0.3 of the HBM rate whatever the expansion cost).
  static constexpr int A_STAGES = BT <= 32 ? 8 : 4;
  static constexpr int FIXED = FP4_WBUF * W_TILE_BYTES + A_STAGES * A_TILE_BYTES;
  static constexpr int MAX_RAW = (BUDGET - FIXED) / FP4_RECORD_BYTES;
  // a multiple of 4 records keeps the tiles behind the ring 1 KiB aligned (4 * 4352 = 17 KiB)
  static constexpr int RAW = (MAX_RAW > 16 ? 16 : MAX_RAW) / 4 * 4;
  // Accumulators: consecutive tcgen05.mma into one accumulator run as a dependent chain (a 128 x 16 x 16 step is
  // latency, not work), so the four k-steps of a k-block go to NACC accumulators BT columns apart, summed in the epilogue.
  static constexpr int NACC_MAX = BT <= 32 ? 4 : (BT <= 128 ? 2 : 1);
  static constexpr int TMEM_COLS = (BT * NACC_MAX) < 32 ? 32 : BT * NACC_MAX;
  static constexpr int DATA_BYTES = RAW * FP4_RECORD_BYTES + FIXED;
  static constexpr int SMEM_BYTES = DATA_BYTES + 1024 + 512;
  static_assert(RAW >= 4, "raw ring too shallow");
  static_assert((RAW * FP4_RECORD_BYTES) % 1024 == 0, "swizzled tiles need 1 KiB alignment");
  static_assert(BT * GEMM_BLOCK_N * 4 <= DATA_BYTES, "the parked fp32 tile must fit in the pipeline memory");
};

__device__ __forceinline__ void fp4_bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// two e2m1 codes (low nibbles of the two halves of `u`) times the block's power-of-two multiplier
__device__ __forceinline__ uint32_t deq_fp4_pair(uint32_t u, __nv_bfloat162 s2) {
  uint32_t t = ((u & 0x00070007u) << 6) | ((u & 0x00080008u) << 12);
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&t);
  v = __hmul2(v, s2);
  return *reinterpret_cast<uint32_t*>(&v);
}

// fp16 form.  A record word holds eight consecutive k values: byte i = (element i in the low nibble, element 4 + i in the
// high nibble).  `cvt.rn.f16x2.e2m1x2` turns a byte into the fp16 pair (element i, element 4 + i); two byte permutes put
// consecutive elements side by side for the K-major tile; one `mul.f16x2` applies the block's power of two.
// the four bytes of a record word -> four fp16x2 registers: byte i = (k value i, k value 4 + i)
__device__ __forceinline__ void cvt_e2m1x8_f16(uint32_t word, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(word));
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
  __half2 v = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&v);
}
// eight codes of a record word -> four fp16x2 registers (consecutive k) times the block's multiplier
__device__ __forceinline__ uint4 deq_fp4_word_f16(uint32_t word, __half2 s2) {
  const uint32_t s = *reinterpret_cast<uint32_t*>(&s2);
  uint32_t h[4];
  cvt_e2m1x8_f16(word, h);       // (k0 k4) (k1 k5) (k2 k6) (k3 k7)
  return make_uint4(hmul2_bits(__byte_perm(h[0], h[1], 0x5410), s), hmul2_bits(__byte_perm(h[2], h[3], 0x5410), s),
                    hmul2_bits(__byte_perm(h[0], h[1], 0x7632), s), hmul2_bits(__byte_perm(h[2], h[3], 0x7632), s));
}

// FP4_WBUF: expanded weight tiles in flight; GROUPS: 1 = all eight expander warps share every k-block (two threads per
// row), 2 = warps 2..5 take the even k-blocks and warps 6..9 the odd ones (one thread per row).
template <int BT, bool HALF, int FP4_WBUF, int GROUPS, int NACC>
__global__ void __launch_bounds__(FP4_THREADS, Fp4Cfg<BT, FP4_WBUF>::TWO_PER_SM ? 2 : 1)
gemm_fp4_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                        const uint8_t* __restrict__ wpacked, int n_tiles_per_expert, int w_by_tma, int skip_rows_le,
                        const GemmParams p) {
  using Cfg = Fp4Cfg<BT, FP4_WBUF>;
  constexpr int RAW = Cfg::RAW;
  constexpr int ARRIVALS = FP4_DEQ_WARPS / GROUPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_ring = smem;
  uint8_t* w_ring = smem + RAW * FP4_RECORD_BYTES;
  uint8_t* a_ring = w_ring + FP4_WBUF * W_TILE_BYTES;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + Cfg::DATA_BYTES);
  uint64_t* raw_empty = raw_full + RAW;
  uint64_t* deq_full = raw_empty + RAW;
  constexpr int A_ST = Cfg::A_STAGES;
  uint64_t* w_empty = deq_full + FP4_WBUF;
  uint64_t* a_full = w_empty + FP4_WBUF;
  uint64_t* a_empty = a_full + A_ST;
  uint64_t* accum_bar = a_empty + A_ST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* use_slot = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  const int num_kb = p.total_kb;
  // The tile list is written by the kernel before this one, so nothing is read ahead of it.
  if (p.pdl) pdl_wait();
  if (m_tile >= *p.grp.num_tiles) return;   // uniform over the CTA
#ifdef OGB_FP4_TRACE
#endif
  const int row0 = p.grp.tile_row0[m_tile];
  const int rows = p.grp.tile_rows[m_tile];
  const int expert = p.grp.tile_expert[m_tile];
  if (rows <= skip_rows_le) return;         // this tile belongs to the streaming kernel below (uniform over the CTA)

  if (threadIdx.x == 0) {
    for (int s = 0; s < RAW; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], ARRIVALS); }
    for (int s = 0; s < FP4_WBUF; ++s) { mbar_init(&deq_full[s], ARRIVALS); mbar_init(&w_empty[s], 1); }
    for (int s = 0; s < A_ST; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl) pdl_launch_dependents();
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer: packed records + activation tiles
      const uint8_t* rec0 = wpacked + (size_t(expert) * num_kb * n_tiles_per_expert + n_tile) * FP4_RECORD_BYTES;
      const size_t rec_stride = size_t(n_tiles_per_expert) * FP4_RECORD_BYTES;
      // A record is 34 rows of 128 bytes: one untiled bulk copy, or (OGB_FP4_TMA=1) one box of a byte tensor map
      const int rec_first = (expert * num_kb) * n_tiles_per_expert + n_tile;
      auto load_raw = [&](int i) {
        const int s = i % RAW;
        mbar_expect_tx(&raw_full[s], FP4_RECORD_BYTES);
        if (w_by_tma) tma_load_2d(raw_ring + s * FP4_RECORD_BYTES, &tmap_w, &raw_full[s], 0, (rec_first + i * n_tiles_per_expert) * (FP4_RECORD_BYTES / 128));
        else fp4_bulk_copy_g2s(raw_ring + s * FP4_RECORD_BYTES, rec0 + size_t(i) * rec_stride, FP4_RECORD_BYTES, &raw_full[s]);
      };
      auto load_a = [&](int i) {
        const int s = i % A_ST;
        mbar_expect_tx(&a_full[s], Cfg::A_TILE_BYTES);
        tma_load_2d(a_ring + s * Cfg::A_TILE_BYTES, &tmap_a, &a_full[s], i * GEMM_BLOCK_K, row0);
      };
      int ri = 0, ai = 0;
      const int pre = min(RAW, num_kb);
      for (; ri < pre; ++ri) load_raw(ri);
      const uint64_t t0 = global_timer_ns();
      uint32_t idle = 0;
      while ((ri < num_kb || ai < num_kb) && !*abort_flag) {
        bool progressed = false;
        if (ri < num_kb && mbar_try_wait(&raw_empty[ri % RAW], ((ri / RAW) & 1) ^ 1)) { load_raw(ri); ++ri; progressed = true; }
        if (ai < num_kb && (ai < A_ST || mbar_try_wait(&a_empty[ai % A_ST], ((ai / A_ST) & 1) ^ 1))) { load_a(ai); ++ai; progressed = true; }
        if (progressed) { idle = 0; continue; }
        if ((++idle & 0x3ff) == 0 && global_timer_ns() - t0 > 4000000000ull) { fail(OGB_ERR_WAIT_TMA); break; }
      }
      if (*abort_flag) {
        volatile int never = 0;
        for (int i = max(0, ri - RAW); i < ri; ++i) mbar_wait_bounded(&raw_full[i % RAW], (i / RAW) & 1, &never, 200000000ull);
        for (int i = max(0, ai - A_ST); i < ai; ++i) mbar_wait_bounded(&a_full[i % A_ST], (i / A_ST) & 1, &never, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = umma_idesc_f16(GEMM_BLOCK_N, BT, HALF ? 0 : 1);   // operand format: fp16 or bf16
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % FP4_WBUF, as = i % A_ST;
        bool got = mbar_wait_bounded(&deq_full[s], (i / FP4_WBUF) & 1, abort_flag);
        got = got && mbar_wait_bounded(&a_full[as], (i / A_ST) & 1, abort_flag);
        if (!got) { fail(OGB_ERR_WAIT_TMA); ok = false; break; }
        tc_fence_after();
        const uint32_t w = smem_u32(w_ring + s * W_TILE_BYTES), a = smem_u32(a_ring + as * Cfg::A_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k)
          umma_f16(tmem_base + uint32_t((k % NACC) * BT), umma_desc_sw128(w + k * GEMM_UMMA_K * 2), umma_desc_sw128(a + k * GEMM_UMMA_K * 2),
                   idesc, (i > 0 || k >= NACC) ? 1u : 0u);
        umma_commit(&w_empty[s]);
        umma_commit(&a_empty[as]);
      }
      if (ok) umma_commit(accum_bar);
    }
  } else {
    // -------------------------------------------------------------- expanders: two threads per weight row of the tile,
    // one block of 32 weights (16 bytes of nibbles, one multiplier byte) each; one arrival per warp on the barriers
    const int dt = threadIdx.x - 64;
    const int row = dt & 127;
    constexpr int WORDS = 4 * GROUPS;                       // 32-bit words of nibbles per thread and k-block
    const int group = GROUPS == 2 ? dt >> 7 : 0;            // which k-blocks this thread expands
    const int part = GROUPS == 2 ? 0 : dt >> 7;             // which block of 32 of the row's 64 weights (GROUPS == 1)
    for (int i = group; i < num_kb; i += GROUPS) {
      const int rs = i % RAW, ws = i % FP4_WBUF;
      bool ok = mbar_wait_bounded(&raw_full[rs], (i / RAW) & 1, abort_flag);
      if (ok && i >= FP4_WBUF) ok = mbar_wait_bounded(&w_empty[ws], ((i / FP4_WBUF) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { fail(OGB_ERR_WAIT_TMA); break; }   // the warp gives up as one (it meets at __syncwarp below)
      const uint8_t* rec = raw_ring + rs * FP4_RECORD_BYTES;
      uint32_t words[WORDS];
#pragma unroll
      for (int h = 0; h < WORDS / 4; ++h) {
        const uint4 q = *reinterpret_cast<const uint4*>(rec + row * 32 + (part + h) * 16);
        words[4 * h] = q.x; words[4 * h + 1] = q.y; words[4 * h + 2] = q.z; words[4 * h + 3] = q.w;
      }
      const uint32_t mul = *reinterpret_cast<const uint16_t*>(rec + GEMM_BLOCK_N * 32 + row * 2);   // exponent fields of the two multipliers
      uint8_t* dst = w_ring + ws * W_TILE_BYTES + row * 128;
      if constexpr (HALF) {
#pragma unroll
        for (int jj = 0; jj < WORDS; ++jj) {
          const int rw = part * 4 + jj;                       // word of the record: (q, b) = (rw / 2, rw % 2)
          const int j = 4 * (rw & 1) + (rw >> 1);             // the 16-byte chunk (8 k values) of the tile row it expands to
          // the stored byte is code + 6; the fp16 exponent field of 2^(code - 127) is code - 112
          const uint32_t m8 = ((rw & 1) ? (mul >> 8) : (mul & 0xFFu)) - 118u;
          const uint32_t sb = (m8 << 10) | (m8 << 26);
          *reinterpret_cast<uint4*>(dst + ((j ^ (row & 7)) << 4)) = deq_fp4_word_f16(words[jj], *reinterpret_cast<const __half2*>(&sb));
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < WORDS; ++jj) {
          const int j = part * 4 + jj;
          const uint32_t m8 = j < 4 ? (mul & 0xFFu) : (mul >> 8);
          const uint32_t sb = (m8 << 7) | (m8 << 23);
          const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&sb);
          uint4 o;
          o.x = deq_fp4_pair(words[jj], s2);
          o.y = deq_fp4_pair(words[jj] >> 4, s2);
          o.z = deq_fp4_pair(words[jj] >> 8, s2);
          o.w = deq_fp4_pair(words[jj] >> 12, s2);
          *reinterpret_cast<uint4*>(dst + ((j ^ (row & 7)) << 4)) = o;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&deq_full[ws]);
        mbar_arrive(&raw_empty[rs]);
      }
    }
  }

  gemm_epilogue<BT, 0>(p, smem, tmem_base, accum_bar, abort_flag, use_slot, n_tile, m_tile, row0, rows, expert * p.N, nullptr, NACC);

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------------------------
// Streaming form for 16-token tiles (decode steps: with 4 of 32 experts per token an expert sees one to a handful of
// tokens).  The kernel above pays the expansion of a whole 128 x 64 tile through shared memory (32 bits of shared-memory
// traffic per 4.25-bit weight, and a chain of four barriers per k-block between its roles) whatever the number of tokens.
// Here the expanded weights never touch shared memory:
//   * One thread streams the packed records, two per stage, through a ring of FP4_STREAM_STAGES bulk copies
//     (asynchronous, tracked by mbarriers: the copies in flight do not depend on what a warp can keep outstanding
//     through its registers).
//   * Each of the eight consumer warps owns 16 weight rows of the record and feeds warp-level `mma.m16n8k16` (fp16 in,
//     fp32 accumulate) straight from registers: a byte of a record word holds the codes of k values i and 4 + i, one
//     `cvt.rn.f16x2.e2m1x2` turns it into an A register, one `mul.f16x2` applies the block's power of two.
//   * The contraction does not care which k value sits in which slot of the instruction as long as both operands agree:
//     lane q = lane % 4 takes the 8 consecutive k values [8 q, 8 q + 8) of each block of 32 (one word of the record), and
//     the activations (up to 8 token rows per pass) are staged in shared memory in the matching order (x0 x4 x1 x5 x2 x6
//     x3 x7 of each group of eight), so a lane's B registers for a block are one 16-byte read.
// The 5th-generation tensor-core instruction cannot take this shape economically: its A operand would have to be written
// to tensor or shared memory first, which is the cost this form exists to avoid.  Tiles of 9..16 rows take a second pass,
// which finds the records in L2.  Every wait is bounded; after a failed wait the warps skip their work but still meet at
// the pass barriers, and the producer waits for its copies in flight before the CTA leaves.
constexpr int FP4_STREAM_CONSUMERS = 8;      // warps 0..7, 16 weight rows each; warp 8 is the producer
constexpr int FP4_STREAM_THREADS = (FP4_STREAM_CONSUMERS + 1) * 32;
constexpr int FP4_STREAM_TOKENS = 8;         // token rows per pass (the N of the instruction)
constexpr int FP4_STREAM_STAGES = 6;         // stages of two records in flight per CTA
constexpr int FP4_STREAM_STAGE_BYTES = 2 * FP4_RECORD_BYTES;
constexpr int FP4_STREAM_MAX_K = 8192;
constexpr int FP4_STREAM_XPAD = 64;          // bytes added to a staged row: the rows of a quarter warp fall on different banks
constexpr int FP4_STREAM_RING_BYTES = FP4_STREAM_STAGES * FP4_STREAM_STAGE_BYTES;
constexpr int FP4_STREAM_RES_BYTES = FP4_STREAM_TOKENS * GEMM_BLOCK_N * 4;
constexpr int FP4_STREAM_FIXED_BYTES = FP4_STREAM_RING_BYTES + FP4_STREAM_RES_BYTES + 256;   // + barriers, abort flag
constexpr int FP4_STREAM_SMEM_MAX = FP4_STREAM_FIXED_BYTES + FP4_STREAM_TOKENS * (FP4_STREAM_MAX_K * 2 + FP4_STREAM_XPAD);

__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__global__ void __launch_bounds__(FP4_STREAM_THREADS, 2)
fp4_stream_grouped_kernel(const void* __restrict__ A_, int lda, const int* __restrict__ row_map, const uint8_t* __restrict__ wpacked,
                          int n_tiles_per_expert, int stage_rows, const GemmParams p) {
  extern __shared__ __align__(128) uint8_t stream_smem[];
  const int K = p.K, num_kb = p.total_kb;
  const int xld = K * 2 + FP4_STREAM_XPAD;                                                  // bytes of a staged row
  uint8_t* ring = stream_smem;                                                               // [STAGES][2][4352]
  float* res = reinterpret_cast<float*>(stream_smem + FP4_STREAM_RING_BYTES);               // [TOKENS][128]
  uint64_t* full = reinterpret_cast<uint64_t*>(stream_smem + FP4_STREAM_RING_BYTES + FP4_STREAM_RES_BYTES);
  uint64_t* empty = full + FP4_STREAM_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + FP4_STREAM_STAGES);
  uint8_t* xs = stream_smem + FP4_STREAM_FIXED_BYTES;                                        // [stage_rows][K / 8 groups][x0 x4 x1 x5 x2 x6 x3 x7]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  if (p.pdl) pdl_wait();                     // the tile list is written by the kernel before this one
  if (m_tile >= *p.grp.num_tiles) return;
  const int rows = p.grp.tile_rows[m_tile];
  if (rows <= 0) return;
  const int row0 = p.grp.tile_row0[m_tile];
  const int expert = p.grp.tile_expert[m_tile];
  if (threadIdx.x == 0) {
    for (int s = 0; s < FP4_STREAM_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], FP4_STREAM_CONSUMERS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (p.pdl) pdl_launch_dependents();
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };

  const int pass_rows = min(FP4_STREAM_TOKENS, stage_rows);
  const int passes = (rows + pass_rows - 1) / pass_rows;
  const int pairs = (num_kb + 1) >> 1;        // stages per pass: two k-blocks each (the last one may hold a single record)
  const uint8_t* rec0 = wpacked + (size_t(expert) * num_kb * n_tiles_per_expert + n_tile) * FP4_RECORD_BYTES;
  const size_t rec_stride = size_t(n_tiles_per_expert) * FP4_RECORD_BYTES;

  if (warp == FP4_STREAM_CONSUMERS) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer
      int issued = 0, s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int pass = 0; pass < passes && ok; ++pass) {
        for (int pr = 0; pr < pairs; ++pr) {
          if (issued >= FP4_STREAM_STAGES) ok = mbar_wait_bounded(&empty[s], phase ^ 1, abort_flag);
          if (!ok) { fail(OGB_ERR_WAIT_TMA); break; }
          const int nk = min(2, num_kb - 2 * pr);
          mbar_expect_tx(&full[s], uint32_t(nk) * FP4_RECORD_BYTES);
          for (int r = 0; r < nk; ++r)
            fp4_bulk_copy_g2s(ring + s * FP4_STREAM_STAGE_BYTES + r * FP4_RECORD_BYTES, rec0 + size_t(2 * pr + r) * rec_stride, FP4_RECORD_BYTES,
                              &full[s]);
          ++issued;
          if (++s == FP4_STREAM_STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {   // nothing of this CTA's shared memory may be handed on while a copy is still landing
        volatile int never = 0;
        for (int i = max(0, issued - FP4_STREAM_STAGES); i < issued; ++i)
          mbar_wait_bounded(&full[i % FP4_STREAM_STAGES], (i / FP4_STREAM_STAGES) & 1, &never, 200000000ull);
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers (256 threads, named barrier 1)
  const int ct = threadIdx.x;                // 0..255
  const int slab = warp * 16;                // rows g and g + 8 of this slab
  const int pair = p.act_pair != 0;
  const int woff = (slab + g) * 32 + q * 8;                  // row g: words (q, 0) and (q, 1); row g + 8 is 256 bytes further
  const int soff = GEMM_BLOCK_N * 32 + (slab + g) * 2;       // the two multiplier bytes of row g; row g + 8 is 16 bytes further
  auto consumer_sync = [] { asm volatile("bar.sync 1, 256;" ::: "memory"); };
  bool ok = true;
  int s = 0;
  uint32_t phase = 0;
  for (int c = 0; c < rows; c += pass_rows) {
    const int nrows = min(pass_rows, rows - c);
    {
      const int groups = K >> 3;             // groups of 8 k values per row
      for (int i = ct; i < pass_rows * groups; i += FP4_STREAM_CONSUMERS * 32) {
        const int t = i / groups, v = i - t * groups;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        if (t < nrows) {
          if (row_map) {
            // the rows were not gathered: sorted row r is row row_map[r] of the bf16 activations, converted here
            const uint4 b = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(A_) + size_t(row_map[row0 + c + t]) * lda + v * 8);
            const float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
            x = make_uint4(pack_f16x2(f0.x, f0.y), pack_f16x2(f1.x, f1.y), pack_f16x2(f2.x, f2.y), pack_f16x2(f3.x, f3.y));
          } else {
            x = *reinterpret_cast<const uint4*>(static_cast<const __half*>(A_) + size_t(row0 + c + t) * lda + v * 8);
          }
        }
        // (x0 x1)(x2 x3)(x4 x5)(x6 x7) -> (x0 x4)(x1 x5)(x2 x6)(x3 x7)
        const uint4 y = make_uint4(__byte_perm(x.x, x.z, 0x5410), __byte_perm(x.x, x.z, 0x7632), __byte_perm(x.y, x.w, 0x5410), __byte_perm(x.y, x.w, 0x7632));
        *reinterpret_cast<uint4*>(xs + size_t(t) * xld + v * 16) = y;
      }
    }
    consumer_sync();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // token g of the pass (rows past the staged ones read row 0: their columns of the product are never stored)
    const uint8_t* xrow = xs + size_t(g < pass_rows ? g : 0) * xld + q * 16;
    for (int pr = 0; pr < pairs; ++pr) {
      ok = ok && mbar_wait_bounded(&full[s], phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int nk = min(2, num_kb - 2 * pr);
      uint2 ca[2], cb[2];
      uint32_t ma[2], mb[2];
      uint4 x0[2], x1[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r < nk) {
          const uint8_t* rec = ring + s * FP4_STREAM_STAGE_BYTES + r * FP4_RECORD_BYTES;
          ca[r] = *reinterpret_cast<const uint2*>(rec + woff);          // .x: block 0, .y: block 1 of row g
          cb[r] = *reinterpret_cast<const uint2*>(rec + woff + 256);    // row g + 8
          ma[r] = *reinterpret_cast<const uint16_t*>(rec + soff);
          mb[r] = *reinterpret_cast<const uint16_t*>(rec + soff + 16);
          x0[r] = *reinterpret_cast<const uint4*>(xrow + (2 * pr + r) * 128);        // block 0
          x1[r] = *reinterpret_cast<const uint4*>(xrow + (2 * pr + r) * 128 + 64);   // block 1
        }
      }
      // the records' bytes are in registers: hand the stage back before the arithmetic
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == FP4_STREAM_STAGES) { s = 0; phase ^= 1; }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r < nk) {
          // the stored byte is code + 6; the fp16 exponent field of 2^(code - 127) is code - 112
          const uint32_t sa0 = ((ma[r] & 0xFFu) - 118u) * 0x04000400u, sa1 = ((ma[r] >> 8) - 118u) * 0x04000400u;
          const uint32_t sb0 = ((mb[r] & 0xFFu) - 118u) * 0x04000400u, sb1 = ((mb[r] >> 8) - 118u) * 0x04000400u;
          uint32_t wa[4], wb[4];
          cvt_e2m1x8_f16(ca[r].x, wa); cvt_e2m1x8_f16(cb[r].x, wb);
          mma_m16n8k16_f16(acc, hmul2_bits(wa[0], sa0), hmul2_bits(wb[0], sb0), hmul2_bits(wa[1], sa0), hmul2_bits(wb[1], sb0), x0[r].x, x0[r].y);
          mma_m16n8k16_f16(acc, hmul2_bits(wa[2], sa0), hmul2_bits(wb[2], sb0), hmul2_bits(wa[3], sa0), hmul2_bits(wb[3], sb0), x0[r].z, x0[r].w);
          cvt_e2m1x8_f16(ca[r].y, wa); cvt_e2m1x8_f16(cb[r].y, wb);
          mma_m16n8k16_f16(acc, hmul2_bits(wa[0], sa1), hmul2_bits(wb[0], sb1), hmul2_bits(wa[1], sa1), hmul2_bits(wb[1], sb1), x1[r].x, x1[r].y);
          mma_m16n8k16_f16(acc, hmul2_bits(wa[2], sa1), hmul2_bits(wb[2], sb1), hmul2_bits(wa[3], sa1), hmul2_bits(wb[3], sb1), x1[r].z, x1[r].w);
        }
      }
    }
    if (!ok && lane == 0) fail(OGB_ERR_WAIT_TMA);
    // accumulator fragment: rows g and g + 8 of the slab, tokens 2 q and 2 q + 1 of the pass
    res[(2 * q) * GEMM_BLOCK_N + slab + g] = acc[0];
    res[(2 * q + 1) * GEMM_BLOCK_N + slab + g] = acc[1];
    res[(2 * q) * GEMM_BLOCK_N + slab + g + 8] = acc[2];
    res[(2 * q + 1) * GEMM_BLOCK_N + slab + g + 8] = acc[3];
    consumer_sync();

    if (*abort_flag == 0) {
      auto store = [&](int m, int col, float v) {
        if (p.out_fp32 == 1) reinterpret_cast<float*>(p.C)[size_t(m) * p.ldc + col] = v;
        else if (p.out_fp32 == 2) reinterpret_cast<__half*>(p.C)[size_t(m) * p.ldc + col] = __float2half_rn(v);
        else reinterpret_cast<__nv_bfloat16*>(p.C)[size_t(m) * p.ldc + col] = __float2bfloat16_rn(v);
      };
      const int bias_off = expert * p.N + n_tile * GEMM_BLOCK_N;
      if (pair) {
        // res[t][0..63] = gate rows, res[t][64..127] = up rows of the same 64 features
        for (int item = ct; item < FP4_STREAM_TOKENS * 64; item += FP4_STREAM_CONSUMERS * 32) {
          const int t = item >> 6, i = item & 63;
          const int col = n_tile * 64 + i;
          if (t < nrows && col < p.N / 2) {
            float gt = res[t * GEMM_BLOCK_N + i], up = res[t * GEMM_BLOCK_N + 64 + i];
            if (p.bias) { gt += bf2f(p.bias[bias_off + i]); up += bf2f(p.bias[bias_off + 64 + i]); }
            float v;
            if (p.act_pair == 1) {
              v = silu(gt) * up;
            } else {
              const float gc = p.act_limit > 0.f ? fminf(gt, p.act_limit) : gt;
              const float uc = p.act_limit > 0.f ? fminf(fmaxf(up, -p.act_limit), p.act_limit) : up;
              v = gc / (1.f + __expf(-p.act_alpha * gc)) * (uc + 1.f);
            }
            store(row0 + c + t, col, v);
          }
        }
      } else {
        for (int item = ct; item < FP4_STREAM_TOKENS * GEMM_BLOCK_N; item += FP4_STREAM_CONSUMERS * 32) {
          const int t = item >> 7, i = item & 127;
          const int col = n_tile * GEMM_BLOCK_N + i;
          if (t < nrows && col < p.N) {
            float v = res[t * GEMM_BLOCK_N + i];
            if (p.bias) v += bf2f(p.bias[bias_off + i]);
            store(row0 + c + t, col, v);
          }
        }
      }
    }
    consumer_sync();   // res and xs are rewritten by the next pass
  }
}

// stage_rows: token rows staged per pass (1..8): an upper bound on the rows of any tile when the host knows one, else 8
static int LaunchFp4Stream(const void* A, int lda, const int* row_map, const uint8_t* wp, int n_tiles, const GemmParams& p, int max_tiles,
                           int stage_rows, cudaStream_t stream) {
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(fp4_stream_grouped_kernel, FP4_STREAM_SMEM_MAX, configured)) return -3;
  const size_t smem = size_t(FP4_STREAM_FIXED_BYTES) + size_t(stage_rows) * (size_t(p.K) * 2 + FP4_STREAM_XPAD);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, max_tiles, 1);
  cfg.blockDim = dim3(FP4_STREAM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, fp4_stream_grouped_kernel, A, lda, row_map, wp, n_tiles, stage_rows, p) == cudaSuccess ? 0 : -4;
}

bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);  // gemm_tcgen05.cu
bool MakeMapBytes128(CUtensorMap* out, const void* ptr, long long rows, int box_rows);          // gemm_tcgen05.cu

template <int BT, bool HALF, int WBUF, int GROUPS, int NACC>
static int LaunchFp4V(const CUtensorMap& ta, const CUtensorMap& tw, int w_by_tma, const uint8_t* wp, int n_tiles, int skip, const GemmParams& p,
                      dim3 grid, cudaStream_t stream) {
  using Cfg = Fp4Cfg<BT, WBUF>;
  static_assert(NACC <= Fp4Cfg<BT, WBUF>::NACC_MAX, "not enough tensor memory for the accumulators");
  auto kern = gemm_fp4_grouped_kernel<BT, HALF, WBUF, GROUPS, NACC>;
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(kern, Cfg::SMEM_BYTES, configured)) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(FP4_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, kern, ta, tw, wp, n_tiles, w_by_tma, skip, p) == cudaSuccess ? 0 : -4;
}

template <int BT, bool HALF>
static int LaunchFp4(const CUtensorMap& ta, const CUtensorMap& tw, int w_by_tma, const uint8_t* wp, int n_tiles, int skip, const GemmParams& p,
                     dim3 grid, cudaStream_t stream) {
  // 16-token tiles: four expanded tiles in flight, the expander warps in two groups that alternate k-blocks, four
  // accumulators; larger tiles: two expanded tiles, one group, one accumulator.  Measured on B200 (gate/up of gpt-oss-20b,
  // 32 tokens): 131 us against 142 us for the single-group forms - the kernel is bound by the rate at which the tensor
  // core retires 128 x 16 x 16 instructions, not by the expansion, the copies or the accumulator chain.
  if constexpr (BT <= 16) return LaunchFp4V<BT, HALF, 4, 2, 4>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
  return LaunchFp4V<BT, HALF, 2, 1, 1>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
}

}  // namespace ogb

using namespace ogb;

// Bytes of the repacked experts: `experts` matrices of [N, K] e2m1 codes (K a multiple of 64; N is padded to 128).
OGB_API long long ogb_fp4_packed_bytes(int experts, int N, int K) {
  return (long long)experts * (K / 64) * ((N + 127) / 128) * FP4_RECORD_BYTES;
}

// Grouped expert GEMM over packed MXFP4 experts; arguments as ogb_moe_gemm with `Wpacked` in the record layout above.
// flags: bit 0 fp32 output, bit 1 paired activation, bit 4 fp16 form (A holds fp16 rows, records in the fp16 layout),
// bit 5 fp16 output.  max_rows_per_tile: an upper bound on the rows of any tile known on the host (the number of tokens
// of the step: an expert receives a token at most once), 0 if unknown.  row_map (or null): A holds the bf16 activations
// [tokens, K] that were NOT gathered, sorted row r is A[row_map[r]] (16-token tiles of the fp16 form only, see
// ogb_moe_fp4_reads_row_map).
// 1 when ogb_moe_gemm_fp4 would take the streaming kernel for this token tile and K (the caller may then skip the row gather)
OGB_API int ogb_moe_fp4_reads_row_map(int token_tile, int K, int half) {
  const char* e = getenv("OGB_FP4_STREAM");
  return (!(e && e[0] == '0') && half && token_tile == 16 && K <= FP4_STREAM_MAX_K && (K % 64) == 0) ? 1 : 0;
}

OGB_API int ogb_moe_gemm_fp4(const void* A, int lda, const void* Wpacked, void* C, int ldc, int rows_total, int N, int K, int experts,
                             const void* bias, int flags, int act_kind, float act_alpha, float act_limit, const int* tile_expert,
                             const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles, int token_tile,
                             int max_rows_per_tile, const int32_t* row_map, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows_total <= 0 || N <= 0 || K <= 0 || experts <= 0 || max_tiles <= 0) return 0;
  if ((K % 64) || (lda % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Wpacked)) & 15) return -1;
  const int act_pair = (flags >> 1) & 1;
  if (act_pair && (N % 128)) return -1;
  if (max_tiles > 65535) return -1;
  static const int pdl_enabled = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  const int bt = token_tile;
  CUtensorMap ta = {};
  if (!row_map && !MakeMapBf16(&ta, A, rows_total, K, lda, bt)) return -2;
  GemmParams p = {};
  p.M = rows_total; p.N = N; p.K = K;
  p.total_kb = K / GEMM_BLOCK_K;
  p.splits = 1; p.kb_per_split = p.total_kb;
  p.C = C; p.ldc = ldc; p.out_fp32 = (flags & 1) ? 1 : ((flags & 32) ? 2 : 0); p.act_pair = act_pair ? act_kind : 0;
  const bool half = (flags & 16) != 0;
  p.act_alpha = act_alpha; p.act_limit = act_limit;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.pdl = pdl_enabled;
  p.grp.tile_expert = tile_expert; p.grp.tile_row0 = tile_row0; p.grp.tile_rows = tile_rows; p.grp.num_tiles = num_tiles;
  const int n_tiles = (N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N;
  CUtensorMap tw = ta;   // unused: records arrive by untiled bulk copies
  const int w_by_tma = 0;
  dim3 grid(n_tiles, max_tiles, 1);
  const uint8_t* wp = static_cast<const uint8_t*>(Wpacked);
  // 16-token tiles of the fp16 form (decode steps) go to the streaming kernel; OGB_FP4_STREAM=0 keeps them on the kernel
  // that expands through shared memory.
  static const int stream_enabled = [] { const char* e = getenv("OGB_FP4_STREAM"); return (e && e[0] == '0') ? 0 : 1; }();
  const int skip = 0;
  if (stream_enabled && half && bt == 16 && K <= FP4_STREAM_MAX_K && max_tiles <= 65535) {
    const int stage_rows = max_rows_per_tile > 0 && max_rows_per_tile < FP4_STREAM_TOKENS ? max_rows_per_tile : FP4_STREAM_TOKENS;
    return LaunchFp4Stream(A, lda, row_map, wp, n_tiles, p, max_tiles, stage_rows, stream);
  }
  if (row_map) return -6;   // only the streaming kernel reads its rows through a map
  switch (bt) {
    case 16: return half ? LaunchFp4<16, true>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream) : LaunchFp4<16, false>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
    case 32: return half ? LaunchFp4<32, true>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream) : LaunchFp4<32, false>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
    case 64: return half ? LaunchFp4<64, true>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream) : LaunchFp4<64, false>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
    case 128: return half ? LaunchFp4<128, true>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream) : LaunchFp4<128, false>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
    case 256: return half ? LaunchFp4<256, true>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream) : LaunchFp4<256, false>(ta, tw, w_by_tma, wp, n_tiles, skip, p, grid, stream);
  }
  return -5;
}
