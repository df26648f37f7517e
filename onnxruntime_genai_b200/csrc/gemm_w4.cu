// Linear layer with int4 block-32 weights (MatMulNBits semantics) on the 5th-generation tensor cores:
//     C[M,N] = A[M,K] * dequant(Wq)[N,K]^T  (+ the shared epilogue of gemm_common.cuh)
//
// Checkpoint semantics (reference: src/python/py/models/builders/base.py:1963-2022,
// quantized_model.py:1017-1107): w[n,k] = (q[n,k] - zero_point[n,k/32]) * scale[n,k/32] with 4-bit q
// and one scale / zero point per block of 32 along K.  The ONNX layout ([N, K/32, 16] bytes + separate
// scale and packed zero-point arrays) is repacked once at load time into tiles that one bulk copy can
// stream: for every (k-block of 64, tile of 128 output rows) a contiguous 5 KiB record
//     [128 rows][32 bytes of nibbles]  +  [128 rows][hi0, lo0|zp0, hi1, lo1|zp1 as 16-bit fields]
// where hi is the block scale rounded to bf16, lo the remainder (scale - hi) as a bf16 whose mantissa needs at most three bits
// for an fp16 scale, and the zero point sits in the four mantissa bits of lo that are always zero: hi + lo is the checkpoint's
// fp16 scale exactly (storing the scale as one bf16 would drop three of its mantissa bits).
// with the nibbles of each 32-bit word ordered so that `(word >> 4j) & 0x000F000F` yields two
// consecutive k values in the two halves of a register (no byte permutes in the inner loop).
//
// Pipeline (192 threads): warp 0 streams the packed records through a deep ring (bulk async copies,
// up to 12-16 records = 60-80 KiB in flight per CTA, the part that has to cover HBM latency) and
// the activation tiles through a 2-deep ring; warps 2..5 (one thread per weight row) turn a record
// into a bf16 K-major tile with the 128-byte swizzle that tcgen05.mma expects
// ((0x4300 | q) is the bf16 number 128 + q, so q - zp is one exact bf16x2 subtract; (q - zp) * lo is exact too (4 + 3 bits),
// and one fused multiply-add with hi rounds (q - zp) * scale to bf16 once); warp 1 issues the MMAs into tensor memory.  HBM traffic is 5 bits per weight.
// Split-K clusters, the SiLU*mul pairing, bias / residual and programmatic dependent launch come
// from the shared epilogue / launch path.  Every wait is bounded.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "gemm_common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int W4_RECORD_BYTES = GEMM_BLOCK_N * 32 + GEMM_BLOCK_N * 8;  // 5120
constexpr int W4_WBUF = 2;                                              // dequantised tiles in flight

template <int BT>
struct W4Cfg {
  static constexpr int A_TILE_BYTES = BT * GEMM_BLOCK_K * 2;
  static constexpr bool TWO_PER_SM = BT <= 64;
  static constexpr int BUDGET = TWO_PER_SM ? 100 * 1024 : 196 * 1024;
  static constexpr int FIXED = W4_WBUF * (W_TILE_BYTES + A_TILE_BYTES);
  static constexpr int MAX_RAW = (BUDGET - FIXED) / W4_RECORD_BYTES;
  static constexpr int RAW = MAX_RAW > 16 ? 16 : MAX_RAW;
  static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  static constexpr int DATA_BYTES = RAW * W4_RECORD_BYTES + FIXED;
  static constexpr int SMEM_BYTES = DATA_BYTES + 1024 + 512;
  static_assert(RAW >= 4, "raw ring too shallow");
  static_assert(BT * GEMM_BLOCK_N * 4 <= DATA_BYTES, "the parked fp32 tile must fit in the pipeline memory");
};

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint32_t deq_pair(uint32_t word, int shift, __nv_bfloat162 z2, __nv_bfloat162 hi2, __nv_bfloat162 lo2) {
  uint32_t t = ((word >> shift) & 0x000F000Fu) | 0x43004300u;  // two bf16 numbers 128 + q
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&t);
  v = __hsub2(v, z2);
  v = __hfma2(v, hi2, __hmul2(v, lo2));                          // round((q - zp) * (hi + lo)) in one rounding
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int BT>
__global__ void __launch_bounds__(GEMM_THREADS, W4Cfg<BT>::TWO_PER_SM ? 2 : 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_a, const uint8_t* __restrict__ wpacked, int n_tiles_total, const GemmParams p) {
  using Cfg = W4Cfg<BT>;
  constexpr int RAW = Cfg::RAW;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw_ring = smem;                                             // [RAW][5120]  (5120 = 5 * 1024: stays 1 KiB aligned)
  uint8_t* w_ring = smem + RAW * W4_RECORD_BYTES;                       // [2][16 KiB] swizzled bf16 weight tiles
  uint8_t* a_ring = w_ring + W4_WBUF * W_TILE_BYTES;                    // [2][BT * 128]
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + Cfg::DATA_BYTES);
  uint64_t* raw_empty = raw_full + RAW;
  uint64_t* deq_full = raw_empty + RAW;
  uint64_t* a_full = deq_full + W4_WBUF;
  uint64_t* w_empty = a_full + W4_WBUF;
  uint64_t* accum_bar = w_empty + W4_WBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* use_slot = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, p.total_kb - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < RAW; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], 128); }
    for (int s = 0; s < W4_WBUF; ++s) { mbar_init(&deq_full[s], 128); mbar_init(&a_full[s], 1); mbar_init(&w_empty[s], 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
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
      auto load_raw = [&](int i) {
        const int s = i % RAW;
        mbar_expect_tx(&raw_full[s], W4_RECORD_BYTES);
        const uint8_t* src = wpacked + (size_t(kb0 + i) * n_tiles_total + n_tile) * W4_RECORD_BYTES;
        bulk_copy_g2s(raw_ring + s * W4_RECORD_BYTES, src, W4_RECORD_BYTES, &raw_full[s]);
      };
      auto load_a = [&](int i) {
        const int s = i % W4_WBUF;
        mbar_expect_tx(&a_full[s], Cfg::A_TILE_BYTES);
        tma_load_2d(a_ring + s * Cfg::A_TILE_BYTES, &tmap_a, &a_full[s], (kb0 + i) * GEMM_BLOCK_K, m_tile * BT);
      };
      int ri = 0, ai = 0;
      const int pre = min(RAW, num_kb);
      for (; ri < pre; ++ri) load_raw(ri);   // weights never depend on an earlier kernel
      if (p.pdl) pdl_wait();
      const uint64_t t0 = global_timer_ns();
      uint32_t idle = 0;
      while ((ri < num_kb || ai < num_kb) && !*abort_flag) {
        bool progressed = false;
        if (ri < num_kb && mbar_try_wait(&raw_empty[ri % RAW], ((ri / RAW) & 1) ^ 1)) { load_raw(ri); ++ri; progressed = true; }
        if (ai < num_kb && (ai < W4_WBUF || mbar_try_wait(&w_empty[ai % W4_WBUF], ((ai / W4_WBUF) & 1) ^ 1))) { load_a(ai); ++ai; progressed = true; }
        if (progressed) { idle = 0; continue; }
        if ((++idle & 0x3ff) == 0 && global_timer_ns() - t0 > 4000000000ull) { fail(OGB_ERR_WAIT_TMA); break; }
      }
      if (*abort_flag) {
        volatile int never = 0;
        for (int i = max(0, ri - RAW); i < ri; ++i) mbar_wait_bounded(&raw_full[i % RAW], (i / RAW) & 1, &never, 200000000ull);
        for (int i = max(0, ai - W4_WBUF); i < ai; ++i) mbar_wait_bounded(&a_full[i % W4_WBUF], (i / W4_WBUF) & 1, &never, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = umma_idesc_f16(GEMM_BLOCK_N, BT, 1);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % W4_WBUF;
        const uint32_t ph = (i / W4_WBUF) & 1;
        if (!mbar_wait_bounded(&deq_full[s], ph, abort_flag) || !mbar_wait_bounded(&a_full[s], ph, abort_flag)) {
          fail(OGB_ERR_WAIT_TMA); ok = false; break;
        }
        tc_fence_after();
        const uint32_t w = smem_u32(w_ring + s * W_TILE_BYTES), a = smem_u32(a_ring + s * Cfg::A_TILE_BYTES);
#pragma unroll
        for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k)
          umma_f16(tmem_base, umma_desc_sw128(w + k * GEMM_UMMA_K * 2), umma_desc_sw128(a + k * GEMM_UMMA_K * 2), idesc,
                   (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&w_empty[s]);
      }
      if (ok) umma_commit(accum_bar);
    }
  } else {
    // -------------------------------------------------------------- dequantisers: thread = weight row of the tile
    const int row = threadIdx.x - 64;
    for (int i = 0; i < num_kb; ++i) {
      const int rs = i % RAW, ws = i % W4_WBUF;
      bool ok = mbar_wait_bounded(&raw_full[rs], (i / RAW) & 1, abort_flag);
      if (ok && i >= W4_WBUF) ok = mbar_wait_bounded(&w_empty[ws], ((i / W4_WBUF) & 1) ^ 1, abort_flag);
      if (!ok) { fail(OGB_ERR_WAIT_TMA); break; }
      const uint8_t* rec = raw_ring + rs * W4_RECORD_BYTES;
      const uint4 q0 = *reinterpret_cast<const uint4*>(rec + row * 32);
      const uint4 q1 = *reinterpret_cast<const uint4*>(rec + row * 32 + 16);
      const uint2 sz = *reinterpret_cast<const uint2*>(rec + GEMM_BLOCK_N * 32 + row * 8);
      const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      uint8_t* dst = w_ring + ws * W_TILE_BYTES + row * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t packed = j < 4 ? sz.x : sz.y;  // (hi, lo | zp) of the 32-block this word belongs to
        const __nv_bfloat16 hi = __ushort_as_bfloat16(uint16_t(packed & 0xFFFF)), lo = __ushort_as_bfloat16(uint16_t((packed >> 16) & 0xFFF0));
        const __nv_bfloat16 zp = __ushort_as_bfloat16(uint16_t(0x4300u | ((packed >> 16) & 0xF)));
        const __nv_bfloat162 hi2 = __halves2bfloat162(hi, hi), lo2 = __halves2bfloat162(lo, lo), z2 = __halves2bfloat162(zp, zp);
        uint4 o;
        o.x = deq_pair(words[j], 0, z2, hi2, lo2);
        o.y = deq_pair(words[j], 4, z2, hi2, lo2);
        o.z = deq_pair(words[j], 8, z2, hi2, lo2);
        o.w = deq_pair(words[j], 12, z2, hi2, lo2);
        *reinterpret_cast<uint4*>(dst + ((j ^ (row & 7)) << 4)) = o;
      }
      fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
      mbar_arrive(&deq_full[ws]);
      mbar_arrive(&raw_empty[rs]);
    }
  }

  gemm_epilogue<BT, 0>(p, smem, tmem_base, accum_bar, abort_flag, use_slot, n_tile, m_tile, m_tile * BT, min(BT, p.M - m_tile * BT), 0);

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// --------------------------------------------------------------------------------- host side
bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);  // gemm_tcgen05.cu

template <int BT>
static int LaunchW4(const CUtensorMap& ta, const uint8_t* wp, int n_tiles_total, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = W4Cfg<BT>;
  auto kern = gemm_w4_kernel<BT>;
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(kern, Cfg::SMEM_BYTES, configured)) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.splits > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = unsigned(p.splits);
    ++na;
  }
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, kern, ta, wp, n_tiles_total, p) == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------- GEMV (1 or 2 tokens)
// Decode of a single sequence (or two): with one or two activation rows the tensor cores have nothing to do and
// the job is to stream the packed weights at HBM speed.  One or two threads per weight row read the nibbles and the
// scale / zero-point pairs of every 64-wide k-block straight from global memory (a warp covers 512 or 1024 contiguous
// bytes), four or eight k-blocks in flight per thread; the activations (and their sums per block of 32, so that
// the zero point costs one multiply per block instead of a subtract per weight) sit in shared memory and are read as
// broadcasts:
//     sum_k (q - z) s x  =  s * (sum_k (128 + q) x  -  (128 + z) * sum_k x)
// The k range is split over a thread-block cluster (up to 8 CTAs) whose partial sums meet in the first CTA's
// shared memory; that CTA adds bias / residual, applies the paired SiLU*mul and stores.
constexpr int GEMV_ROWS = 128;     // weight rows per CTA (one packed record per k-block)
constexpr int GEMV_MAX_KB = 32;    // k-blocks per CTA held as activations in shared memory (x: MT * 64 * 4 bytes each)

// TPR = threads per weight row: 1 (each thread takes both blocks of 32 of a k-block; launches with many CTAs) or 2 (one
// block of 32 each: twice the threads and loads in flight, for launches whose CTAs alone cannot fill the GPU).
template <int MT, int TPR>
__global__ void __launch_bounds__(GEMV_ROWS * TPR)
gemv_w4_kernel(const __nv_bfloat16* __restrict__ A, int lda, const uint8_t* __restrict__ wpacked, int n_tiles_total, const GemmParams p) {
  constexpr int THREADS = GEMV_ROWS * TPR;
  constexpr int HB = 2 / TPR;                   // blocks of 32 per thread and k-block
  constexpr int GEMV_AHEAD = 4 * TPR;           // k-blocks in flight per thread (32 or 16 bytes each)
  __shared__ __align__(16) float xs[MT][GEMV_MAX_KB * 64];
  __shared__ float xsum[MT][GEMV_MAX_KB * 2];
  __shared__ float part[MT][GEMV_ROWS];         // this CTA's partial sums, read by the first CTA of the cluster
  const int tid = threadIdx.x;
  const int row = tid / TPR, half = tid % TPR;  // weight row of the tile; first block of 32 of each k-block for this thread
  const int n_tile = blockIdx.x, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int num_kb = max(0, min(p.kb_per_split, p.total_kb - kb0));
  const uint8_t* rec0 = wpacked + (size_t(kb0) * n_tiles_total + n_tile) * W4_RECORD_BYTES;
  const size_t rec_stride = size_t(n_tiles_total) * W4_RECORD_BYTES;

  // Weights first, before the wait on the previous kernel (nothing earlier in the stream writes them): several k-blocks
  // per thread are in flight at any time, which is what covers the HBM latency of this short kernel.
  uint4 nb[GEMV_AHEAD][HB];
  uint32_t szq[GEMV_AHEAD][HB];
  auto fetch = [&](int kb, int slot) {
    const uint8_t* r = rec0 + size_t(kb) * rec_stride;
#pragma unroll
    for (int h = 0; h < HB; ++h) {
      const int hh = half * HB + h;
      nb[slot][h] = *reinterpret_cast<const uint4*>(r + row * 32 + hh * 16);
      szq[slot][h] = *reinterpret_cast<const uint32_t*>(r + GEMM_BLOCK_N * 32 + row * 8 + hh * 4);
    }
  };
#pragma unroll
  for (int a = 0; a < GEMV_AHEAD; ++a)
    if (a < num_kb) fetch(a, a);
  if (p.pdl) { pdl_launch_dependents(); pdl_wait(); }

  // stage the activations of this k range as fp32 and their sums per block of 32 (one warp per block, shuffle reduction)
  for (int i = tid; i < num_kb * 64; i += THREADS) {
#pragma unroll
    for (int m = 0; m < MT; ++m) xs[m][i] = m < p.M ? bf2f(A[size_t(m) * lda + size_t(kb0) * 64 + i]) : 0.f;
  }
  __syncthreads();
  for (int b = tid >> 5; b < num_kb * 2 * MT; b += THREADS / 32) {
    const int m = b / (num_kb * 2), blk = b % (num_kb * 2);
    const float t = warp_sum(xs[m][blk * 32 + (tid & 31)]);
    if ((tid & 31) == 0) xsum[m][blk] = t;
  }
  __syncthreads();

  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;

  for (int kb0i = 0; kb0i < num_kb; kb0i += GEMV_AHEAD) {
#pragma unroll
    for (int a = 0; a < GEMV_AHEAD; ++a) {
      const int kb = kb0i + a;
      if (kb >= num_kb) break;
      uint4 nib[HB];
      float2 sc[HB];
#pragma unroll
      for (int h = 0; h < HB; ++h) {     // (scale = hi + lo, 128 + zero point)
        nib[h] = nb[a][h];
        const uint32_t pk = szq[a][h];
        sc[h].x = __uint_as_float(pk << 16) + __uint_as_float(pk & 0xFFF00000u);
        sc[h].y = __uint_as_float(0x43000000u | ((pk & 0x000F0000u)));
      }
      if (kb + GEMV_AHEAD < num_kb) fetch(kb + GEMV_AHEAD, a);     // refill the slot just consumed
#pragma unroll
      for (int h = 0; h < HB; ++h) {
        const int hh = half * HB + h;
        const uint32_t words[4] = {nib[h].x, nib[h].y, nib[h].z, nib[h].w};
        float dot[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) dot[m] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w = words[j];
          float q[8];
#pragma unroll
          for (int pr = 0; pr < 4; ++pr) {
            const uint32_t t = ((w >> (4 * pr)) & 0x000F000Fu) | 0x43004300u;   // two bf16 numbers 128 + q
            q[2 * pr] = __uint_as_float(t << 16);
            q[2 * pr + 1] = __uint_as_float(t & 0xFFFF0000u);
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[m][kb * 64 + hh * 32 + j * 8]);
            const float4 xb = *reinterpret_cast<const float4*>(&xs[m][kb * 64 + hh * 32 + j * 8 + 4]);
            dot[m] += q[0] * xa.x + q[1] * xa.y + q[2] * xa.z + q[3] * xa.w + q[4] * xb.x + q[5] * xb.y + q[6] * xb.z + q[7] * xb.w;
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] += sc[h].x * (dot[m] - sc[h].y * xsum[m][kb * 2 + hh]);
      }
    }
  }
  if (TPR == 2) {   // the two threads of a row
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], 1);
  }

  if (half == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) part[m][row] = acc[m];
  }
  if (p.splits > 1) cluster_sync_all(); else __syncthreads();

  if (split == 0) {
    const bool pair = p.act_pair != 0;
    const int n_out = pair ? p.N / 2 : p.N;
    const uint32_t part_addr = smem_u32(&part[0][0]);
    auto total = [&](int m, int row) {
      float t = 0.f;
      for (int s = 0; s < p.splits; ++s) {
        if (p.splits > 1) {
          float v;
          const uint32_t ra = dsmem_addr(part_addr + uint32_t(m * GEMV_ROWS + row) * 4, uint32_t(s));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
          t += v;
        } else {
          t += part[m][row];
        }
      }
      const int n = n_tile * GEMM_BLOCK_N + row;
      if (p.bias && n < p.N) t += bf2f(p.bias[n]);
      return t;
    };
    const int rows_out = pair ? 64 : GEMV_ROWS;
    if (tid < rows_out) {
      const int col = pair ? n_tile * 64 + tid : n_tile * GEMM_BLOCK_N + tid;
      if (col < n_out) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m >= p.M) break;
          float v = total(m, tid);
          if (pair) v = silu(v) * total(m, tid + 64);
          if (p.residual) v += bf2f(p.residual[size_t(m) * p.ldr + col]);
          if (p.out_fp32) reinterpret_cast<float*>(p.C)[size_t(m) * p.ldc + col] = v;
          else reinterpret_cast<__nv_bfloat16*>(p.C)[size_t(m) * p.ldc + col] = f2bf(v);
        }
      }
    }
  }
  if (p.splits > 1) cluster_sync_all();   // peers keep their shared memory alive until the first CTA has read it
}

template <int MT, int TPR>
static int LaunchGemvW4(const __nv_bfloat16* A, int lda, const uint8_t* wp, int n_tiles_total, const GemmParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles_total, 1, p.splits);
  cfg.blockDim = dim3(GEMV_ROWS * TPR);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.splits > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = unsigned(p.splits);
    ++na;
  }
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, gemv_w4_kernel<MT, TPR>, A, lda, wp, n_tiles_total, p) == cudaSuccess ? 0 : -4;
}

}  // namespace ogb

using namespace ogb;

// Bytes of the repacked weight for an [N, K] int4 matrix (K a multiple of 64; N is padded to 128).
OGB_API long long ogb_w4_packed_bytes(int N, int K) {
  return (long long)(K / 64) * ((N + 127) / 128) * W4_RECORD_BYTES;
}

// flags: bit 0 fp32 output, bit 1 paired silu(gate)*up epilogue (rows interleaved in blocks of 64 before packing).
OGB_API int ogb_gemm_w4(const void* A, int lda, const void* Wpacked, void* C, int ldc, int M, int N, int K, const void* bias,
                        const void* residual, int ldr, int flags, int splits, int* status, int sm_count, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 64) || (lda % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(Wpacked) & 15)) return -1;
  const int out_fp32 = flags & 1, act_pair = (flags >> 1) & 1;
  if (act_pair && (N % 128)) return -1;
  static const int pdl_enabled = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  const int bt = ogb_gemm_token_tile(M, 0);
  const int n_tiles = (N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N, m_tiles = (M + bt - 1) / bt;
  const int total_kb = K / GEMM_BLOCK_K;
  static const int gemv_enabled = [] { const char* e = getenv("OGB_W4_GEMV"); return (e && e[0] == '0') ? 0 : 1; }();
  if (M <= 2 && gemv_enabled && total_kb <= 8 * GEMV_MAX_KB) {
    // a few tokens: stream the weights with one thread per row, k split over a cluster sized to fill the GPU
    int gs = splits > 0 ? splits : 1;
    if (splits <= 0) while (gs < 8 && n_tiles * gs < 4 * sm_count && total_kb / (gs * 2) >= 2) gs *= 2;
    if (gs > 8) gs = 8;
    while ((total_kb + gs - 1) / gs > GEMV_MAX_KB) gs *= 2;
    if (gs > total_kb) gs = total_kb;
    int per = (total_kb + gs - 1) / gs;
    while (gs > 1 && per * (gs - 1) >= total_kb) { --gs; per = (total_kb + gs - 1) / gs; }
    if (gs <= 8 && per <= GEMV_MAX_KB) {
      GemmParams g = {};
      g.M = M; g.N = N; g.K = K; g.splits = gs; g.kb_per_split = per; g.total_kb = total_kb;
      g.C = C; g.ldc = ldc; g.out_fp32 = out_fp32; g.act_pair = act_pair;
      g.residual = static_cast<const __nv_bfloat16*>(residual); g.ldr = ldr;
      g.bias = static_cast<const __nv_bfloat16*>(bias);
      g.status = status; g.pdl = pdl_enabled;
      const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(A);
      const uint8_t* w = static_cast<const uint8_t*>(Wpacked);
      const bool wide = n_tiles * gs < 2 * sm_count;   // few CTAs: two threads per row double the loads in flight
      if (M == 1) return wide ? LaunchGemvW4<1, 2>(a, lda, w, n_tiles, g, stream) : LaunchGemvW4<1, 1>(a, lda, w, n_tiles, g, stream);
      return wide ? LaunchGemvW4<2, 2>(a, lda, w, n_tiles, g, stream) : LaunchGemvW4<2, 1>(a, lda, w, n_tiles, g, stream);
    }
  }
  if (splits <= 0) {
    // Every k-block costs a dequantisation pass on top of the copy, so the k range is cut finer than for bf16 weights:
    // the largest power of two that keeps 8 k-blocks per CTA and all CTAs resident at once.
    const int slots = (bt <= 64 ? 2 : 1) * sm_count;
    splits = 1;
    for (int s2 = 2; s2 <= 8; s2 *= 2) {
      if (s2 > bt || total_kb / s2 < 8 || n_tiles * m_tiles * s2 > slots) break;
      splits = s2;
    }
  }
  if (splits > 8) splits = 8;
  if (splits > bt) splits = bt;
  if (splits > total_kb) splits = total_kb;
  int kb_per = (total_kb + splits - 1) / splits;
  while (splits > 1 && kb_per * (splits - 1) >= total_kb) { --splits; kb_per = (total_kb + splits - 1) / splits; }
  CUtensorMap ta;
  if (!MakeMapBf16(&ta, A, M, K, lda, bt)) return -2;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.splits = splits; p.kb_per_split = kb_per; p.total_kb = total_kb;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.act_pair = act_pair;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.pdl = pdl_enabled;
  dim3 grid(n_tiles, m_tiles, splits);
  const uint8_t* wp = static_cast<const uint8_t*>(Wpacked);
  switch (bt) {
    case 16: return LaunchW4<16>(ta, wp, n_tiles, p, grid, stream);
    case 32: return LaunchW4<32>(ta, wp, n_tiles, p, grid, stream);
    case 64: return LaunchW4<64>(ta, wp, n_tiles, p, grid, stream);
    case 128: return LaunchW4<128>(ta, wp, n_tiles, p, grid, stream);
    case 256: return LaunchW4<256>(ta, wp, n_tiles, p, grid, stream);
  }
  return -5;
}
