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
// activations converted to fp16 by the row gather (and by the gate/up epilogue for the down projection), the
// nibbles stay in their natural order and `cvt.rn.f16x2.e2m1x2` expands two codes per instruction; the multiplier
// byte is then the fp16 exponent field of 2^(scale - 127), scale - 112.  One conversion and one multiply per pair
// of weights instead of six integer / bf16 operations: the expansion stops being the limit of the weight stream.
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
// bytes at the full rate).  The way past this limit is to put the weights on the instruction's N side (256 rows per
// instruction, tokens padded to M = 64), which changes the accumulator layout and the epilogue; not done here.
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

// four bytes of e2m1 pairs (low nibble = first element) -> four fp16x2 registers times the block's multiplier
__device__ __forceinline__ uint4 deq_fp4_word_f16(uint32_t word, __half2 s2) {
  uint32_t h0, h1, h2, h3;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(word));
  auto mul = [&](uint32_t h) {
    __half2 v = __hmul2(*reinterpret_cast<__half2*>(&h), s2);
    return *reinterpret_cast<uint32_t*>(&v);
  };
  return make_uint4(mul(h0), mul(h1), mul(h2), mul(h3));
}

// FP4_WBUF: expanded weight tiles in flight; GROUPS: 1 = all eight expander warps share every k-block (two threads per
// row), 2 = warps 2..5 take the even k-blocks and warps 6..9 the odd ones (one thread per row).
template <int BT, bool HALF, int FP4_WBUF, int GROUPS, int NACC>
__global__ void __launch_bounds__(FP4_THREADS, Fp4Cfg<BT, FP4_WBUF>::TWO_PER_SM ? 2 : 1)
gemm_fp4_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                        const uint8_t* __restrict__ wpacked, int n_tiles_per_expert, int w_by_tma, const GemmParams p) {
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
          const int j = part * 4 + jj;
          const uint32_t m8 = j < 4 ? (mul & 0xFFu) : (mul >> 8);
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

bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);  // gemm_tcgen05.cu
bool MakeMapBytes128(CUtensorMap* out, const void* ptr, long long rows, int box_rows);          // gemm_tcgen05.cu

template <int BT, bool HALF, int WBUF, int GROUPS, int NACC>
static int LaunchFp4V(const CUtensorMap& ta, const CUtensorMap& tw, int w_by_tma, const uint8_t* wp, int n_tiles, const GemmParams& p, dim3 grid,
                      cudaStream_t stream) {
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
  return cudaLaunchKernelEx(&cfg, kern, ta, tw, wp, n_tiles, w_by_tma, p) == cudaSuccess ? 0 : -4;
}

template <int BT, bool HALF>
static int LaunchFp4(const CUtensorMap& ta, const CUtensorMap& tw, int w_by_tma, const uint8_t* wp, int n_tiles, const GemmParams& p, dim3 grid,
                     cudaStream_t stream) {
  // 16-token tiles: four expanded tiles in flight, the expander warps in two groups that alternate k-blocks, four
  // accumulators; larger tiles: two expanded tiles, one group, one accumulator.  Measured on B200 (gate/up of gpt-oss-20b,
  // 32 tokens): 131 us against 142 us for the single-group forms - the kernel is bound by the rate at which the tensor
  // core retires 128 x 16 x 16 instructions, not by the expansion, the copies or the accumulator chain.
  if constexpr (BT <= 16) return LaunchFp4V<BT, HALF, 4, 2, 4>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
  return LaunchFp4V<BT, HALF, 2, 1, 1>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
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
// of the step: an expert receives a token at most once), 0 if unknown (not used by the kernel selection).
OGB_API int ogb_moe_gemm_fp4(const void* A, int lda, const void* Wpacked, void* C, int ldc, int rows_total, int N, int K, int experts,
                             const void* bias, int flags, int act_kind, float act_alpha, float act_limit, const int* tile_expert,
                             const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles, int token_tile,
                             int max_rows_per_tile, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows_total <= 0 || N <= 0 || K <= 0 || experts <= 0 || max_tiles <= 0) return 0;
  if ((K % 64) || (lda % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Wpacked)) & 15) return -1;
  const int act_pair = (flags >> 1) & 1;
  if (act_pair && (N % 128)) return -1;
  if (max_tiles > 65535) return -1;
  static const int pdl_enabled = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  const int bt = token_tile;
  CUtensorMap ta;
  if (!MakeMapBf16(&ta, A, rows_total, K, lda, bt)) return -2;
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
  switch (bt) {
    case 16: return half ? LaunchFp4<16, true>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream) : LaunchFp4<16, false>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
    case 32: return half ? LaunchFp4<32, true>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream) : LaunchFp4<32, false>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
    case 64: return half ? LaunchFp4<64, true>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream) : LaunchFp4<64, false>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
    case 128: return half ? LaunchFp4<128, true>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream) : LaunchFp4<128, false>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
    case 256: return half ? LaunchFp4<256, true>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream) : LaunchFp4<256, false>(ta, tw, w_by_tma, wp, n_tiles, p, grid, stream);
  }
  return -5;
}
