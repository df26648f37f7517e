// bf16 linear layer on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T  (+ epilogue)
//
// The weight is the UMMA "M" operand (128 output features per CTA) and the activations are the
// UMMA "N" operand (16..256 tokens), so the same kernel serves decode (few tokens, bandwidth bound:
// every SM streams weight tiles through a deep TMA pipeline, split-K fills the machine when N/128
// is small) and prefill (256-token tiles, compute bound).  Both operands are K-major in shared
// memory with the 128-byte swizzle written by TMA; accumulators live in tensor memory and are read
// back with tcgen05.ld by four epilogue warps.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane),
// warps 2..5 = epilogue (warp 2 also owns the TMEM allocation).
//
// Epilogues: optional bias[N], optional residual add, fp32 or bf16 output, and a dual-accumulator
// mode that computes silu(A*Wg^T) * (A*Wu^T) for a stacked [gate; up] weight (reference graph:
// gate_proj/up_proj MatMul + Sigmoid/Mul, src/python/py/models/builders/base.py:4065-4131).
// Split-K partial tiles go to a caller-provided fp32 workspace; the CTA that arrives last at the
// tile's counter reduces them in a fixed order (deterministic) and runs the epilogue.
//
// Every mbarrier wait is bounded: when one runs out the kernel records a status code, waits
// (bounded) for its own TMA copies in flight, frees its tensor memory and returns.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int GEMM_BLOCK_N = 128;
constexpr int GEMM_BLOCK_K = 64;
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int W_TILE_BYTES = GEMM_BLOCK_N * GEMM_BLOCK_K * 2;  // 16 KiB

struct GemmParams {
  int M, N, K;
  int dual_row_offset;  // rows between the gate tile and the up tile (dual mode)
  int splits, kb_per_split, total_kb;
  void* C;
  int ldc;
  int out_fp32;
  const __nv_bfloat16* residual;
  int ldr;
  const __nv_bfloat16* bias;
  float* workspace;
  int* counters;
  int* status;
};

template <int BT, bool DUAL>
struct GemmCfg {
  static constexpr int A_TILE_BYTES = BT * GEMM_BLOCK_K * 2;
  static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * W_TILE_BYTES + A_TILE_BYTES;
  static constexpr int MAX_STAGES = (196 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int TMEM_COLS_RAW = (DUAL ? 2 : 1) * BT;
  static constexpr int TMEM_COLS = TMEM_COLS_RAW < 32 ? 32 : TMEM_COLS_RAW;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

template <int BT, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, GemmParams p) {
  using Cfg = GemmCfg<BT, DUAL>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, p.total_kb - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
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

  auto stage_w0 = [&](int s) { return smem + s * Cfg::STAGE_BYTES; };
  auto stage_w1 = [&](int s) { return smem + s * Cfg::STAGE_BYTES + W_TILE_BYTES; };
  auto stage_a = [&](int s) { return smem + s * Cfg::STAGE_BYTES + (DUAL ? 2 : 1) * W_TILE_BYTES; };
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      int issued = 0;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); break; }
        mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
        const int kx = (kb0 + i) * GEMM_BLOCK_K;
        tma_load_2d(stage_w0(s), &tmap_w, &full_bar[s], kx, n_tile * GEMM_BLOCK_N);
        if (DUAL) tma_load_2d(stage_w1(s), &tmap_w, &full_bar[s], kx, p.dual_row_offset + n_tile * GEMM_BLOCK_N);
        tma_load_2d(stage_a(s), &tmap_a, &full_bar[s], kx, m_tile * BT);
        ++issued;
      }
      if (*abort_flag) {
        // Copies already issued still write this CTA's shared memory: give them time to land.
        volatile int never = 0;
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait_bounded(&full_bar[i % STAGES], (i / STAGES) & 1, &never, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = umma_idesc_f16(GEMM_BLOCK_N, BT, 1);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag)) { fail(OGB_ERR_WAIT_TMA); ok = false; break; }
        tc_fence_after();
        const uint32_t w0 = smem_u32(stage_w0(s)), w1 = smem_u32(stage_w1(s)), a = smem_u32(stage_a(s));
#pragma unroll
        for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k) {
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          const uint64_t db = umma_desc_sw128(a + k * GEMM_UMMA_K * 2);
          umma_f16(tmem_base, umma_desc_sw128(w0 + k * GEMM_UMMA_K * 2), db, idesc, acc);
          if (DUAL) umma_f16(tmem_base + BT, umma_desc_sw128(w1 + k * GEMM_UMMA_K * 2), db, idesc, acc);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(accum_bar);
    }
  } else {
    // -------------------------------------------------------------------- epilogue (4 warps)
    const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
    const int row = quarter * 32 + lane;
    const int n = n_tile * GEMM_BLOCK_N + row;
    const bool n_ok = n < p.N;
    const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
    if (!mbar_wait_bounded(accum_bar, 0, abort_flag, 4000000000ull)) fail(OGB_ERR_WAIT_MMA);
    // Make the decision uniform over the 128 epilogue threads: they meet at named barriers below.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool have = (*abort_flag == 0);
    tc_fence_after();

    const float bias0 = (p.bias && n_ok) ? bf2f(p.bias[n]) : 0.f;
    const float bias1 = (DUAL && p.bias && n_ok) ? bf2f(p.bias[p.dual_row_offset + n]) : 0.f;
    auto emit = [&](int m, float g, float u) {
      float v = g + bias0;
      if (DUAL) v = silu(v) * (u + bias1);
      if (p.residual) v += bf2f(p.residual[size_t(m) * p.ldr + n]);
      if (p.out_fp32) reinterpret_cast<float*>(p.C)[size_t(m) * p.ldc + n] = v;
      else reinterpret_cast<__nv_bfloat16*>(p.C)[size_t(m) * p.ldc + n] = f2bf(v);
    };

    if (have) {
      const size_t plane = size_t(p.M) * p.N;  // one fp32 plane of the split-K workspace
      float* ws = p.workspace + (size_t(split) * (DUAL ? 2 : 1)) * plane;
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 16) {
        uint32_t r0[16], r1[16];
        tmem_ld16(taddr + c0, r0);
        if (DUAL) tmem_ld16(taddr + BT + c0, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m_tile * BT + c0 + j;
          if (m < p.M && n_ok) {
            const float g = __uint_as_float(r0[j]);
            const float u = DUAL ? __uint_as_float(r1[j]) : 0.f;
            if (p.splits == 1) emit(m, g, u);
            else {
              ws[size_t(m) * p.N + n] = g;
              if (DUAL) ws[plane + size_t(m) * p.N + n] = u;
            }
          }
        }
      }
      if (p.splits > 1) {
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int tile_id = m_tile * gridDim.x + n_tile;
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&p.counters[tile_id], 1);
          *last_flag = (prev == p.splits - 1);
          if (prev == p.splits - 1) p.counters[tile_id] = 0;  // self-cleaning for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          const int m_end = min(p.M, (m_tile + 1) * BT);
          if (n_ok) {
            for (int m = m_tile * BT; m < m_end; ++m) {
              float g = 0.f, u = 0.f;
              for (int s = 0; s < p.splits; ++s) {
                const float* w = p.workspace + (size_t(s) * (DUAL ? 2 : 1)) * plane;
                g += __ldcg(&w[size_t(m) * p.N + n]);
                if (DUAL) u += __ldcg(&w[plane + size_t(m) * p.N + n]);
              }
              emit(m, g, u);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// --------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn GetEncodeTiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr; int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ size_t(v);
    return h;
  }
};

// 2-D bf16 row-major tensor [rows, cols] (leading dimension ld elements), box = [box_rows, 64],
// 128-byte swizzle, out-of-range elements read as zero.
static bool MakeMap(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn enc = GetEncodeTiled();
  if (!enc) return false;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  cuuint32_t box[2] = {cuuint32_t(GEMM_BLOCK_K), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

template <int BT, bool DUAL>
static int Launch(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BT, DUAL>;
  static bool configured = false;
  auto kern = gemm_tcgen05_kernel<BT, DUAL>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -3;
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tw, ta, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_gemm_token_tile(int M, int dual) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128 || dual) return 128;
  return 256;
}

// Number of split-K partitions the launcher picks for a problem (workspace sizing helper).
OGB_API int ogb_gemm_auto_splits(int M, int N, int K, int dual, int sm_count) {
  const int bt = ogb_gemm_token_tile(M, dual);
  const int tiles = ((N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N) * ((M + bt - 1) / bt);
  const int total_kb = (K + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  if (tiles >= sm_count || total_kb < 8) return 1;
  int splits = (sm_count + tiles / 2) / tiles;          // round to the nearest whole wave
  splits = splits < 1 ? 1 : splits;
  const int max_by_k = total_kb / 4 > 0 ? total_kb / 4 : 1;  // keep >= 4 k-blocks per split
  if (splits > max_by_k) splits = max_by_k;
  if (splits > 16) splits = 16;
  return splits;
}

OGB_API int ogb_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                          const void* bias, const void* residual, int ldr, int out_fp32, int dual, int dual_row_offset,
                          int splits, void* workspace, long long workspace_bytes, int* counters, int num_counters,
                          int* status, int sm_count, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return -1;  // 16-byte global strides for TMA
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  const int bt = ogb_gemm_token_tile(M, dual);
  const int n_tiles = (N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N, m_tiles = (M + bt - 1) / bt;
  const int total_kb = (K + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  if (splits <= 0) splits = ogb_gemm_auto_splits(M, N, K, dual, sm_count);
  if (splits > total_kb) splits = total_kb;
  // shrink until the workspace and the counters fit
  while (splits > 1 && (size_t(splits) * (dual ? 2 : 1) * size_t(M) * N * 4 > size_t(workspace_bytes) || n_tiles * m_tiles > num_counters || !workspace || !counters))
    --splits;
  int kb_per = (total_kb + splits - 1) / splits;
  splits = (total_kb + kb_per - 1) / kb_per;  // no empty split

  const int w_rows = dual ? dual_row_offset + N : N;
  CUtensorMap tw, ta;
  if (!MakeMap(&tw, W, w_rows, K, ldw, GEMM_BLOCK_N)) return -2;
  if (!MakeMap(&ta, A, M, K, lda, bt)) return -2;

  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.dual_row_offset = dual_row_offset;
  p.splits = splits; p.kb_per_split = kb_per; p.total_kb = total_kb;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.workspace = static_cast<float*>(workspace); p.counters = counters; p.status = status;
  dim3 grid(n_tiles, m_tiles, splits);
#define OGB_GEMM_CASE(BT_)                                                         \
  case BT_: return dual ? Launch<BT_, true>(tw, ta, p, grid, stream) : Launch<BT_, false>(tw, ta, p, grid, stream);
  switch (bt) {
    OGB_GEMM_CASE(16)
    OGB_GEMM_CASE(32)
    OGB_GEMM_CASE(64)
    OGB_GEMM_CASE(128)
    case 256: return Launch<256, false>(tw, ta, p, grid, stream);
  }
#undef OGB_GEMM_CASE
  return -5;
}
