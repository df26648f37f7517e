// Linear layer with int4 block-32 weights (MatMulNBits semantics) on the 5th-generation tensor cores:
//     C[M,N] = A[M,K] * dequant(Wq)[N,K]^T  (+ the shared epilogue of gemm_common.cuh)
//
// Checkpoint semantics (reference: src/python/py/models/builders/base.py:1963-2022,
// quantized_model.py:1017-1107): w[n,k] = (q[n,k] - zero_point[n,k/32]) * scale[n,k/32] with 4-bit q
// and one scale / zero point per block of 32 along K.  The ONNX layout ([N, K/32, 16] bytes + separate
// scale and packed zero-point arrays) is repacked once at load time into tiles that one bulk copy can
// stream: for every (k-block of 64, tile of 128 output rows) a contiguous 5 KiB record
//     [128 rows][32 bytes of nibbles]  +  [128 rows][scale0, 128+zp0, scale1, 128+zp1 as bf16]
// with the nibbles of each 32-bit word ordered so that `(word >> 4j) & 0x000F000F` yields two
// consecutive k values in the two halves of a register (no byte permutes in the inner loop).
//
// Pipeline (192 threads): warp 0 streams the packed records through a deep ring (bulk async copies,
// up to 12-16 records = 60-80 KiB in flight per CTA, the part that has to cover HBM latency) and
// the activation tiles through a 2-deep ring; warps 2..5 (one thread per weight row) turn a record
// into a bf16 K-major tile with the 128-byte swizzle that tcgen05.mma expects
// ((0x4300 | q) is the bf16 number 128 + q, so (q - zp) * scale is one exact bf16x2 subtract and one
// multiply); warp 1 issues the MMAs into tensor memory.  HBM traffic is 5 bits per weight.
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

__device__ __forceinline__ uint32_t deq_pair(uint32_t word, int shift, __nv_bfloat162 z2, __nv_bfloat162 s2) {
  uint32_t t = ((word >> shift) & 0x000F000Fu) | 0x43004300u;  // two bf16 numbers 128 + q
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&t);
  v = __hmul2(__hsub2(v, z2), s2);
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
        const uint32_t packed = j < 4 ? sz.x : sz.y;  // (scale, 128 + zp) of the 32-block this word belongs to
        const __nv_bfloat16 sc = __ushort_as_bfloat16(uint16_t(packed & 0xFFFF)), zp = __ushort_as_bfloat16(uint16_t(packed >> 16));
        const __nv_bfloat162 s2 = __halves2bfloat162(sc, sc), z2 = __halves2bfloat162(zp, zp);
        uint4 o;
        o.x = deq_pair(words[j], 0, z2, s2);
        o.y = deq_pair(words[j], 4, z2, s2);
        o.z = deq_pair(words[j], 8, z2, s2);
        o.w = deq_pair(words[j], 12, z2, s2);
        *reinterpret_cast<uint4*>(dst + ((j ^ (row & 7)) << 4)) = o;
      }
      fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's async proxy
      mbar_arrive(&deq_full[ws]);
      mbar_arrive(&raw_empty[rs]);
    }
  }

  gemm_epilogue<BT>(p, smem, tmem_base, accum_bar, abort_flag, use_slot, n_tile, m_tile, m_tile * BT, min(BT, p.M - m_tile * BT), 0);

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// --------------------------------------------------------------------------------- host side
bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows);  // gemm_tcgen05.cu

template <int BT>
static int LaunchW4(const CUtensorMap& ta, const uint8_t* wp, int n_tiles_total, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = W4Cfg<BT>;
  static bool configured = false;
  auto kern = gemm_w4_kernel<BT>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
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
  if (splits <= 0) splits = ogb_gemm_auto_splits(M, N, K, 0, sm_count);
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
