// bf16 linear layer on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T  (+ epilogue),
// optionally fused with the tensor-parallel all-reduce of the partial sums over NVLink.
//
// The weight is the UMMA "M" operand (128 output features per CTA) and the activations are the
// UMMA "N" operand (16..256 tokens), so the same kernel serves decode (few tokens, bandwidth bound:
// every SM streams weight tiles through a deep TMA pipeline, two CTAs per SM) and prefill
// (256-token tiles, compute bound).  Both operands are K-major in shared memory with the 128-byte
// swizzle written by TMA; accumulators live in tensor memory and are read back with tcgen05.ld.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane),
// warps 2..5 = epilogue (warp 2 also owns the TMEM allocation).
//
// Split-K (decode: N/128 tiles alone cannot fill 148 SMs) runs as a thread-block CLUSTER of up to
// 8 CTAs along z: each CTA accumulates its K slice in its own tensor memory and parks the fp32 tile
// in its (by then idle) pipeline shared memory; after a cluster barrier every CTA reduces a slice
// of the token columns by reading its peers' tiles through distributed shared memory in rank order
// (deterministic).  No global workspace, no atomics.  The same shared-memory tile transposes the
// accumulator (one thread per output feature) into 16-byte row segments for the stores.
//
// Programmatic dependent launch: the producer prefetches WEIGHT tiles (which no earlier kernel
// writes) for every pipeline stage before griddepcontrol.wait; activations, residual reads and all
// stores come after it, so weight streaming overlaps the tail of the previous kernel.
//
// Epilogues: bias[N], residual add, fp32 or bf16 output, and a paired activation for the MLP: with
// the gate and up projection rows interleaved in blocks of 64 (tile t = 64 gate rows then the 64
// up rows of the same features) the kernel writes silu(gate) * up, N/2 columns (reference graph:
// gate_proj/up_proj MatMul + Sigmoid/Mul, src/python/py/models/builders/base.py:4065-4131).
//
// Tensor-parallel all-reduce (row-parallel o_proj / down_proj in decode), fused: instead of
// storing its reduced slice, a CTA pushes it (bf16) into the receive buffer of EVERY rank with
// 16-byte peer stores over NVLink that carry the call's flag next to the data, then collects
// (bounded waits on the flags) the same slice of every rank from its local buffer, sums in rank
// order (bit-identical on every rank), adds the residual and stores.  No fence, no separate
// arrival flag, no barrier between ranks: one NVLink write latency per all-reduce.  Buffers
// alternate by the parity of a call counter kept on the device, so the kernel replays unchanged
// inside CUDA graphs.  The reference has no distributed code at all; the comparison bar is
// GEMM + ncclAllReduce.
//
// Every wait is bounded: when one runs out the kernel records a status code, waits (bounded) for
// its own TMA copies in flight, still meets its barriers, frees its tensor memory and returns.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "gemm_common.cuh"
#include "kernels.h"

namespace ogb {

template <int BT, int COMM, bool DEEP>
__global__ void __launch_bounds__(GEMM_THREADS, GemmCfg<BT, DEEP>::TWO_PER_SM ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  using Cfg = GemmCfg<BT, DEEP>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* use_slot = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);
  float* ssq = reinterpret_cast<float*>(smem + Cfg::SSQ_OFFSET);   // [BT] sums of squares of the activation rows (folded norm)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, p.total_kb - kb0);
  // Grouped mode: the tile list is written by the kernel before this one, so nothing is read ahead of it.
  const bool grouped = p.grp.tile_expert != nullptr;
  int row0 = m_tile * BT, rows = min(BT, p.M - row0), w_row0 = 0;
  if (grouped) {
    if (p.pdl) pdl_wait();
    if (m_tile >= *p.grp.num_tiles) return;   // uniform over the CTA and over its split-K cluster
    row0 = p.grp.tile_row0[m_tile];
    rows = p.grp.tile_rows[m_tile];
    w_row0 = p.grp.tile_expert[m_tile] * p.N;
  }

  const bool gather = p.ag_rows > 0;
  const bool norm = p.norm_eps > 0.f;   // warps 2..5 read every activation tile too: a stage is empty once they have as well
  if (threadIdx.x == 0) {
    // gathered activations: a stage is full when the weight tile has landed AND the 128 assembling threads have arrived
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], gather ? 1 + 128 : 1); mbar_init(&empty_bar[s], norm ? 1 + 4 : 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_a);
  }
  constexpr uint32_t tmem_cols = Cfg::TMEM_COLS;
  if (warp == 2) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl) pdl_launch_dependents();

  auto stage_w = [&](int s) { return smem + s * Cfg::STAGE_BYTES; };
  auto stage_a = [&](int s) { return smem + s * Cfg::STAGE_BYTES + W_TILE_BYTES; };
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      auto load_w = [&](int i) {
        const int s = i % STAGES;
        mbar_expect_tx(&full_bar[s], gather ? W_TILE_BYTES : Cfg::STAGE_BYTES);
        tma_load_2d(stage_w(s), &tmap_w, &full_bar[s], (kb0 + i) * GEMM_BLOCK_K, w_row0 + n_tile * GEMM_BLOCK_N);
      };
      auto load_a = [&](int i) {
        if (gather) return;   // assembled by warps 2..5 below
        tma_load_2d(stage_a(i % STAGES), &tmap_a, &full_bar[i % STAGES], (kb0 + i) * GEMM_BLOCK_K, row0);
      };
      // Weights are never written by an earlier kernel of the stream: fill the pipeline with them
      // before waiting for the producer of the activations.
      const int pre = min(STAGES, num_kb);
      for (int i = 0; i < pre; ++i) load_w(i);
      if (p.pdl) pdl_wait();
      if (COMM != 0) *use_slot = comm_open_call(p.comm, gridDim.x * gridDim.y * gridDim.z);
      for (int i = 0; i < pre; ++i) load_a(i);
      int issued = pre;
      for (int i = pre; i < num_kb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); break; }
        load_w(i);
        load_a(i);
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
        const uint32_t w = smem_u32(stage_w(s)), a = smem_u32(stage_a(s));
#pragma unroll
        for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k)
          umma_f16(tmem_base, umma_desc_sw128(w + k * GEMM_UMMA_K * 2), umma_desc_sw128(a + k * GEMM_UMMA_K * 2), idesc,
                   (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(accum_bar);
    }
  }

  if (gather && warp >= 2) {
    // ------------------------------------------------------------------ all-gather -> GEMM: assemble the activation tiles
    // Each k-block's [BT rows][64] tile is built from 16-byte lines {4 bf16, flag} of the local receive buffer (written by
    // every rank's push in the previous fused call), waiting for each line's flag, and stored in the 128-byte-swizzled
    // K-major layout the tensor core reads; then the 128 threads arrive on the stage's barrier.
    const int gt = threadIdx.x - 64;
    if (p.pdl) pdl_wait();
    const uint32_t ep = *reinterpret_cast<volatile uint32_t*>(p.comm.epoch) - 1u;   // the push was the previous call
    const uint32_t flag = comm_flag(ep);
    const size_t plane_lines = size_t(p.comm.plane_elems) / 4;
    const uint4* base = p.comm.buf[p.comm.rank] + size_t(ep & 1) * p.comm.world * plane_lines;
    bool dead = *reinterpret_cast<volatile int*>(p.status) != 0;
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES && !mbar_wait_bounded(&empty_bar[s], ((i / STAGES) & 1) ^ 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); }
      uint8_t* tile = stage_a(s);
      const int k0 = (kb0 + i) * GEMM_BLOCK_K;
      for (int idx = gt; idx < BT * 16; idx += 128) {
        const int r = idx >> 4, ln = idx & 15;          // row of the tile, line of the row (4 bf16 each)
        const int m = row0 + r, k = k0 + ln * 4;
        uint2 d = make_uint2(0u, 0u);
        if (r < rows && k < p.K) {
          const int owner = m / p.ag_rows, rl = m - owner * p.ag_rows;
          const uint4 q = wait_line(base + size_t(owner) * plane_lines + (size_t(rl) * p.K + k) / 4, flag, dead, p.status);
          d = make_uint2(q.x, q.z);
        }
        const int chunk = ln >> 1;
        *reinterpret_cast<uint2*>(tile + r * 128 + (((chunk ^ (r & 7)) << 4) | ((ln & 1) << 3))) = d;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to tcgen05.mma
      mbar_arrive(&full_bar[s]);
    }
    if (dead) *abort_flag = 1;
  }

  if (norm && warp >= 2) {
    // ------------------------------------------------------------------ folded RMS norm: sum of squares of every activation row
    // The four epilogue warps (idle during the main loop) read each activation tile from shared memory once it has landed.  A
    // row's 128 bytes are contiguous whatever the swizzle, so 16-byte chunk c of the tile belongs to row c / 8; thread t takes
    // chunks t, t + 128, ...  Eight neighbouring threads share a row and combine at the end.
    constexpr int CHUNKS = BT * 8, PER = (CHUNKS + 127) / 128;
    const int t = threadIdx.x - 64;
    float acc[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) acc[k] = 0.f;
    for (int i = 0; i < num_kb; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait_bounded(&full_bar[s], (i / STAGES) & 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); break; }
      const uint8_t* tile = stage_a(s);
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int c = t + 128 * k;
        if (c < CHUNKS) {
          const uint4 q = *reinterpret_cast<const uint4*>(tile + c * 16);
          const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
          acc[k] += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + cc.x * cc.x + cc.y * cc.y + d.x * d.x + d.y * d.y;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      float v = acc[k];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      const int c = t + 128 * k;
      if ((t & 7) == 0 && c < CHUNKS) ssq[c >> 3] = v;
    }
  }

  gemm_epilogue<BT, COMM>(p, smem, tmem_base, accum_bar, abort_flag, use_slot, n_tile, m_tile, row0, rows, w_row0, norm ? ssq : nullptr);

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, tmem_cols);
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

// A byte buffer seen as rows of 128 bytes, box = [box_rows, 128], no swizzle: one box is box_rows * 128 contiguous bytes in
// global and in shared memory (the packed weight records of gemm_fp4.cu).
bool MakeMapBytes128(CUtensorMap* out, const void* ptr, long long rows, int box_rows) {
  EncodeTiledFn enc = GetEncodeTiled();
  if (!enc || rows <= 0 || rows > 0x7fffffffll || box_rows > 256) return false;
  cuuint64_t dims[2] = {128, cuuint64_t(rows)};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {128, cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Shared with gemm_w4.cu (activation tensor maps).
bool MakeMapBf16(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  return MakeMap(out, ptr, rows, cols, ld, box_rows);
}

template <int BT, int COMM, bool DEEP>
static int LaunchC(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BT, DEEP>;
  auto kern = gemm_tcgen05_kernel<BT, COMM, DEEP>;
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
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = unsigned(p.splits);
    ++na;
  }
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, kern, tw, ta, p) == cudaSuccess ? 0 : -4;
}

static int ogb_sm_count_current() {
  static int n = 0;
  if (n == 0) { int dev = 0; if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148; }
  return n;
}

// One kernel instantiation per token tile and per reduction form: the local form does not carry the reductions' code.
template <int BT>
static int Launch(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  // deep pipeline, one CTA per SM: decode-sized launches that put at most one CTA on an SM anyway
  if constexpr (BT <= 64) {
    static const int deep_env = [] { const char* e = getenv("OGB_GEMM_DEEP"); return e ? atoi(e) : -1; }();
    const bool deep = deep_env != 0;      // OGB_GEMM_DEEP=0: always the two-CTAs-per-SM form
    if (deep && (long long)grid.x * grid.y * grid.z <= ogb_sm_count_current()) {
      if (!p.comm_epilogue) return LaunchC<BT, 0, true>(tw, ta, p, grid, stream);
      if (!p.nvls) return LaunchC<BT, 1, true>(tw, ta, p, grid, stream);
    }
  }
  if (!p.comm_epilogue) return LaunchC<BT, 0, false>(tw, ta, p, grid, stream);
  return p.nvls ? LaunchC<BT, 2, false>(tw, ta, p, grid, stream) : LaunchC<BT, 1, false>(tw, ta, p, grid, stream);
}

// How many split-K clusters of `splits` CTAs of the decode kernel the device can hold at once (0: the query failed).  The
// CTAs of a cluster must sit in one GPC, so this is less than (resident CTAs) / splits in general.
template <int BT>
static int MaxActiveClusters(int splits) {
  using Cfg = GemmCfg<BT>;
  auto kern = gemm_tcgen05_kernel<BT, 0, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, unsigned(splits));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = unsigned(splits);
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

// ------------------------------------------------------------------------------------------ persistent prefill kernel
// Compute-bound shapes (hundreds of tokens and more): one CTA per SM walks a list of 128 x 256 output tiles, weight-tile
// index slowest so that the CTAs of the moment share a few weight tiles and the whole activation matrix in L2.  The TMA
// producer streams k-blocks across tile boundaries without draining the ring; the accumulator is double buffered in
// tensor memory (2 x 256 columns), so the MMA warp starts the next tile while the four epilogue warps drain the previous
// one (tcgen05.ld, 16 token columns at a time through a small staging tile that pairs gate / up rows and makes the
// stores 16-byte row segments).  Same epilogues as the other kernel except split-K and the collectives, which prefill
// does not use.
constexpr int PERS_BT = 256;
constexpr int PERS_STAGES = 4;
constexpr int PERS_STAGE_BYTES = W_TILE_BYTES + PERS_BT * GEMM_BLOCK_K * 2;       // 16 KiB + 32 KiB
constexpr int PERS_STAGING_BYTES = 2 * 16 * GEMM_BLOCK_N * 4;                     // two [16][128] fp32 chunks
constexpr int PERS_SMEM_BYTES = PERS_STAGES * PERS_STAGE_BYTES + PERS_STAGING_BYTES + 1024 + 256;

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, const GemmParams p,
                               int n_tiles, int m_tiles) {
  constexpr int BT = PERS_BT, STAGES = PERS_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* staging = reinterpret_cast<float*>(smem + STAGES * PERS_STAGE_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * PERS_STAGE_BYTES + PERS_STAGING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;     // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;          // [2] epilogue (128 arrivals) -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_abort = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = n_tiles * m_tiles;
  const int num_kb = p.total_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    *abort_flag = 0;
    *epi_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_a);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.pdl) pdl_launch_dependents();
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };
  auto stage_w = [&](int s) { return smem + s * PERS_STAGE_BYTES; };
  auto stage_a = [&](int s) { return smem + s * PERS_STAGE_BYTES + W_TILE_BYTES; };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer: k-blocks of all my tiles, back to back
      bool waited = false;
      int it = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const int n_tile = t / m_tiles, m_tile = t % m_tiles;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait_bounded(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); break; }
          mbar_expect_tx(&full_bar[s], PERS_STAGE_BYTES);
          tma_load_2d(stage_w(s), &tmap_w, &full_bar[s], kb * GEMM_BLOCK_K, n_tile * GEMM_BLOCK_N);
          if (!waited) {               // the first weight tile may go out before the previous kernel has finished; activations may not
            if (p.pdl) pdl_wait();
            waited = true;
          }
          tma_load_2d(stage_a(s), &tmap_a, &full_bar[s], kb * GEMM_BLOCK_K, m_tile * BT);
        }
      }
      if (*abort_flag) {   // copies already issued still write this CTA's shared memory: give them time to land
        volatile int never = 0;
        for (int i = max(0, it - STAGES); i < it; ++i) mbar_wait_bounded(&full_bar[i % STAGES], (i / STAGES) & 1, &never, 200000000ull);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer: alternate the two accumulators
      constexpr uint32_t idesc = umma_idesc_f16(GEMM_BLOCK_N, BT, 1);
      int it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++j) {
        const int buf = j & 1;
        if (j >= 2 && !mbar_wait_bounded(&acc_empty[buf], ((j >> 1) & 1) ^ 1, abort_flag)) { fail(OGB_ERR_WAIT_MMA); ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + uint32_t(buf * BT);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_bounded(&full_bar[s], (it / STAGES) & 1, abort_flag)) { fail(OGB_ERR_WAIT_TMA); ok = false; break; }
          tc_fence_after();
          const uint32_t w = smem_u32(stage_w(s)), a = smem_u32(stage_a(s));
#pragma unroll
          for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k)
            umma_f16(acc, umma_desc_sw128(w + k * GEMM_UMMA_K * 2), umma_desc_sw128(a + k * GEMM_UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue warps 2..5
    const int et = threadIdx.x - 64;
    const int quarter = warp & 3;            // TMEM lanes this warp may read
    const int row = quarter * 32 + lane;     // weight row of the tile held by this thread
    const bool pair = p.act_pair != 0;
    const int OCT = pair ? 8 : 16;
    const int n_out = pair ? p.N / 2 : p.N;
    if (p.pdl) pdl_wait();                   // residual reads and all stores come after the previous kernel
    int j = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++j) {
      const int buf = j & 1;
      const int n_tile = t / m_tiles, m_tile = t % m_tiles;
      // a failed wait is published in a word only the epilogue threads write, before the barrier: all 128 take the same branch
      if (!mbar_wait_bounded(&acc_full[buf], (j >> 1) & 1, abort_flag, 4000000000ull)) { fail(OGB_ERR_WAIT_MMA); *epi_abort = 1; }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*epi_abort) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * BT);
      const int col0 = n_tile * (pair ? 64 : 128);
      for (int c0 = 0, ch = 0; c0 < BT; c0 += 16, ++ch) {
        float* part = staging + (ch & 1) * 16 * GEMM_BLOCK_N;      // [16 token columns][128 weight rows]
        uint32_t r0[16];
        tmem_ld16(taddr + c0, r0);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 16; ++q) part[q * GEMM_BLOCK_N + row] = __uint_as_float(r0[q]);
        asm volatile("bar.sync 1, 128;" ::: "memory");             // chunk visible; the other buffer is free again after the NEXT sync
        for (int item = et; item < 16 * OCT; item += 128) {
          const int mc = item / OCT, oc = item % OCT;
          const int m = m_tile * BT + c0 + mc;
          if (m >= p.M) continue;
          float v[8];
          const float* src = part + mc * GEMM_BLOCK_N + oc * 8;
#pragma unroll
          for (int q = 0; q < 8; ++q) v[q] = src[q];
          if (p.bias) {
#pragma unroll
            for (int q = 0; q < 8; ++q) if (n_tile * GEMM_BLOCK_N + oc * 8 + q < p.N) v[q] += bf2f(p.bias[n_tile * GEMM_BLOCK_N + oc * 8 + q]);
          }
          if (pair) {
            float u[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) u[q] = src[64 + q];
            if (p.bias) {
#pragma unroll
              for (int q = 0; q < 8; ++q) u[q] += bf2f(p.bias[n_tile * GEMM_BLOCK_N + 64 + oc * 8 + q]);
            }
            if (p.act_pair == 1) {
#pragma unroll
              for (int q = 0; q < 8; ++q) v[q] = silu(v[q]) * u[q];
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float g = p.act_limit > 0.f ? fminf(v[q], p.act_limit) : v[q];
                const float w = p.act_limit > 0.f ? fminf(fmaxf(u[q], -p.act_limit), p.act_limit) : u[q];
                v[q] = g / (1.f + __expf(-p.act_alpha * g)) * (w + 1.f);
              }
            }
          }
          const int col = col0 + oc * 8;
          if (col >= n_out) continue;
          if (p.residual) {
#pragma unroll
            for (int q = 0; q < 8; ++q) if (col + q < n_out) v[q] += bf2f(p.residual[size_t(m) * p.ldr + col + q]);
          }
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + size_t(m) * p.ldc + col;
            if (col + 8 <= n_out && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
              *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
              *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q) if (col + q < n_out) dst[q] = v[q];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(m) * p.ldc + col;
            if (col + 8 <= n_out && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q) if (col + q < n_out) dst[q] = f2bf(v[q]);
            }
          }
        }
      }
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, 512);
}

static int LaunchPersistent(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, int n_tiles, int m_tiles, int sm_count,
                            cudaStream_t stream) {
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(gemm_tcgen05_persistent_kernel, PERS_SMEM_BYTES, configured)) return -3;
  const int tiles = n_tiles * m_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(tiles < sm_count ? tiles : sm_count));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = PERS_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_tcgen05_persistent_kernel, tw, ta, p, n_tiles, m_tiles) == cudaSuccess ? 0 : -4;
}

}  // namespace ogb

using namespace ogb;

// Per-device registration of the symmetric buffers used by the fused all-reduce.
static CommParams g_comm[16] = {};

namespace ogb {
const CommParams* ogb_comm_params(int device) { return (device >= 0 && device < 16) ? &g_comm[device] : nullptr; }
}  // namespace ogb

OGB_API int ogb_gemm_token_tile(int M, int dual) {
  (void)dual;
  // prefill-sized problems: 256-token tiles, one CTA per SM
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

// Number of split-K partitions (cluster size along z: 1, 2, 4 or 8).  Every CTA of the launch must fit on the GPU at once
// (two resident CTAs per SM for decode-sized tiles).  Up to 4 partitions pay off as soon as each keeps two k-blocks: the
// epilogue of a tile (one thread per 8 outputs, fetched cold) is divided between the cluster's CTAs, which matters more than
// the short main loops.  Launches of at most one CTA per SM run a pipeline twice as deep (one CTA per SM: o 13.0 -> 12.2 us).
// Measured on B200 at 64 tokens, us per launch (benchmark/kernel_case.py --gemm_splits; rows marked tpN are the per-rank
// shapes of N-way tensor parallelism with the fused all-reduce talking to itself):
//   qkv  (N 6144, K 4096):  s=2 16.8  s=4 15.5  s=8 25.8 (a second wave from 288 CTAs on)
//   o    (N 4096, K 4096):  s=2 15.8  s=4 12.9  s=8 14.7
//   down (N 4096, K 14336): s=2 41.3  s=4 28.4  s=8 27.6
//   tp8 o    (N 4096, K 512):  s=1 15.7  s=2 11.6  s=4 10.2  s=8 12.9      tp8 qkv     (N 768,  K 4096): s=1 24.1  s=4 9.8   s=8 8.6
//   tp8 down (N 4096, K 1792): s=1 21.7  s=2 14.9  s=4 12.2  s=8 14.4      tp4 gate/up (N 7168, K 4096): s=2 17.9  s=4 16.7  s=8 25.3
//   tp2 down (N 4096, K 7168): s=1 47.6  s=2 28.8  s=4 20.7  s=8 20.4      tp2 gate/up (N 14336, K 4096): s=1 29.2 s=2 23.8  s=4 32.8
// Reducing through global memory instead of the cluster's shared memory (partials in an fp32 scratch, the last CTA of a
// tile sums them) was measured too and is not kept: o 22.5..29.7, qkv 24.3..27.6, down 38.6..45.5 us.
OGB_API int ogb_gemm_auto_splits(int M, int N, int K, int dual, int sm_count) {
  const int bt = ogb_gemm_token_tile(M, dual);
  const int tiles = ((N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N) * ((M + bt - 1) / bt);
  const int total_kb = (K + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  const int slots = (bt <= 128 ? 2 : 1) * sm_count;
  int best = 1;
  for (int s = 2; s <= 8; s *= 2) {
    if (s > bt || tiles * s > slots) break;
    const int kbs = total_kb / s;
    // 8 partitions: long k ranges whose 4-way split would not fit one CTA per SM (that form runs the deep pipeline: down
    // 25.1 us at s=4 against 27.7 at s=8), or launches so small that even 8 partitions leave one CTA per SM
    const bool ok = s <= 4 ? kbs >= 2 : ((kbs >= 16 && tiles * 4 > sm_count) || (tiles * s <= sm_count && kbs >= 8));
    if (ok) best = s;
  }
  return best;
}

OGB_API int ogb_gemm_max_active_clusters(int bt, int splits) {
  if (splits < 1 || splits > 8) return 0;
  switch (bt) {
    case 16: return MaxActiveClusters<16>(splits);
    case 32: return MaxActiveClusters<32>(splits);
    case 64: return MaxActiveClusters<64>(splits);
    case 128: return MaxActiveClusters<128>(splits);
  }
  return 0;
}

// Registers this rank's view of the symmetric buffers (peer-mapped pointers) for a device.
// buf[r]: rank r's receive buffer as mapped into this process, 2 * world * plane_elems * 4 bytes, zero-initialised
// (flagged lines: every 8 payload bytes travel in a 16-byte line); epoch: two local zero-initialised words.
// world = 0 unregisters.
OGB_API int ogb_comm_register(int device, int world, int rank, void** buf, void* epoch, long long plane_elems) {
  if (device < 0 || device >= 16 || world < 0 || world > COMM_MAX_WORLD || (plane_elems % 8)) return -1;
  CommParams c = {};
  c.world = world; c.rank = rank; c.plane_elems = plane_elems;
  for (int r = 0; r < world; ++r) c.buf[r] = static_cast<uint4*>(buf[r]);
  c.epoch = static_cast<uint32_t*>(epoch);
  g_comm[device] = c;
  return 0;
}

// Adds the NVLS (NVSwitch multicast) buffers to a registered device: `data` / `out` are this rank's two planes of
// 2 * plane_elems bf16 each inside a symmetric allocation, `ctr` 2 * NV_MAX_CTAS zero-initialised words in it; the *_mc
// pointers are the same ranges through the allocation's multicast mapping; `expected` is 2 * NV_MAX_CTAS local
// zero-initialised words.  data == nullptr removes them (the flagged-line kernels serve again).
OGB_API int ogb_comm_register_nvls(int device, void* data, void* data_mc, void* out, void* out_mc, void* ctr, void* ctr_mc, void* expected,
                                   long long plane_elems) {
  if (device < 0 || device >= 16 || (plane_elems % 8)) return -1;
  CommParams& c = g_comm[device];
  if (data && (c.world < 1 || !data_mc || !out || !out_mc || !ctr || !ctr_mc || !expected)) return -1;
  c.nv_data = static_cast<__nv_bfloat16*>(data); c.nv_data_mc = static_cast<__nv_bfloat16*>(data_mc);
  c.nv_out = static_cast<__nv_bfloat16*>(out); c.nv_out_mc = static_cast<__nv_bfloat16*>(out_mc);
  c.nv_ctr = static_cast<uint32_t*>(ctr); c.nv_ctr_mc = static_cast<uint32_t*>(ctr_mc);
  c.nv_expected = static_cast<uint32_t*>(expected);
  c.nv_plane_elems = data ? plane_elems : 0;
  return 0;
}

// Process-wide choices of the fused reductions: [0] use NVLS when registered (default: OGB_TP_NVLS == 1; off otherwise - measured
// on B200 the multimem round trips cost more than flagged lines at decode sizes, 36 against 24 us for GEMM + all-reduce at two
// ranks), [1] byte count
// (world * tensor bytes) above which the NVLS all-reduce takes the two-shot form (default: OGB_NVLS_TWO_SHOT_BYTES or 2 MiB),
// [2] flagged-line all-reduce in two hops: 1 yes, 0 no, -1 from 4 ranks up (default: OGB_AR_TWO_SHOT or -1).
static long long g_comm_opts[3] = {-1, -1, -2};
namespace ogb {
const long long* ogb_comm_options() {
  if (g_comm_opts[0] < 0) { const char* e = getenv("OGB_TP_NVLS"); g_comm_opts[0] = (e && e[0] == '1') ? 1 : 0; }
  if (g_comm_opts[1] < 0) { const char* e = getenv("OGB_NVLS_TWO_SHOT_BYTES"); g_comm_opts[1] = e ? atoll(e) : (2ll << 20); }
  if (g_comm_opts[2] < -1) { const char* e = getenv("OGB_AR_TWO_SHOT"); g_comm_opts[2] = e ? atoi(e) : -1; }
  return g_comm_opts;
}
}  // namespace ogb
// A negative value leaves an option as it is (p2p_two_hop: -2 leaves it, -1 is its automatic setting).
OGB_API int ogb_comm_set_options(int use_nvls, long long two_shot_bytes, int p2p_two_hop) {
  ogb_comm_options();
  if (use_nvls >= 0) g_comm_opts[0] = use_nvls ? 1 : 0;
  if (two_shot_bytes >= 0) g_comm_opts[1] = two_shot_bytes;
  if (p2p_two_hop >= -1) g_comm_opts[2] = p2p_two_hop;
  return 0;
}

// 1 when the NVLS buffers of `device` are registered, 2 when the reductions also use them (option [0]).
OGB_API int ogb_comm_has_nvls(int device) {
  if (!(device >= 0 && device < 16 && g_comm[device].nv_data_mc != nullptr)) return 0;
  return ogb_comm_options()[0] ? 2 : 1;
}

// Elements (bf16) that one fused reduction may cover on `device`: the NVLS plane when registered, else the flagged-line plane.
OGB_API long long ogb_comm_capacity(int device) {
  if (device < 0 || device >= 16 || g_comm[device].world < 1) return 0;
  return g_comm[device].nv_data_mc ? g_comm[device].nv_plane_elems : g_comm[device].plane_elems;
}

// flags bit 0: fp32 output; bit 1: paired silu(gate)*up epilogue (N = 2 * output columns, rows
// interleaved in blocks of 64); bit 2: fused all-reduce over the registered symmetric buffers; bit 3: fused
// reduce-scatter by token rows instead (rank r ends up with rows [r * ceil(M / world), ...) of the sum, written as
// rows 0.. of C; residual, if given, is that slice too); bit 4: activations gathered from the ranks' pushes.
OGB_API int ogb_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                          const void* bias, const void* residual, int ldr, int flags, int splits, int device, int* status,
                          int sm_count, void* stream_) {
  return ogb_gemm_bf16_fused(A, lda, W, ldw, C, ldc, M, N, K, bias, residual, ldr, flags, splits, device, status, sm_count, stream_, nullptr);
}

// ogb_gemm_bf16 with the decode-step fusions of `f` (see OgbGemmFused in kernels.h; nullptr: none):
//  * norm_eps > 0: A holds un-normalised rows and W carries the RMS norm's weight; row m of the product is multiplied by
//    rsqrt(mean(A[m]^2) + norm_eps) before bias and activation (SimplifiedLayerNormalization folded into its consumer);
//  * positions != nullptr: QKV projection with rotary embedding and KV-cache append in the epilogue: C [M, Hq * D] receives
//    the rotated queries only, keys (rotated) and values go to row slots[m] of the caches.  Needs 128 % D == 0, rot % 16 == 0,
//    N == (Hq + 2 * Hkv) * D, bf16 caches, and excludes the reductions, fp32 output and the paired activation.
OGB_API int ogb_gemm_bf16_fused(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                const void* bias, const void* residual, int ldr, int flags, int splits, int device, int* status,
                                int sm_count, void* stream_, const OgbGemmFused* f) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return -1;  // 16-byte global strides for TMA
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  const int out_fp32 = flags & 1, act_pair = (flags >> 1) & 1, fused_rs = (flags >> 3) & 1, fused_ar = ((flags >> 2) & 1) | fused_rs;
  if (act_pair && (N % 128)) return -1;
  static const int pdl_enabled = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  const int bt = ogb_gemm_token_tile(M, 0);
  const int n_tiles = (N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N, m_tiles = (M + bt - 1) / bt;
  const int total_kb = (K + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  const bool auto_split = splits <= 0;      // an explicit split count asks for the (tiles x k-splits) kernel
  if (splits <= 0) splits = ogb_gemm_auto_splits(M, N, K, 0, sm_count);
  if (splits > 8) splits = 8;          // portable cluster size
  if (splits > bt) splits = bt;        // every cluster rank finishes at least one token column
  if (splits > total_kb) splits = total_kb;
  int kb_per = (total_kb + splits - 1) / splits;
  while (splits > 1 && kb_per * (splits - 1) >= total_kb) { --splits; kb_per = (total_kb + splits - 1) / splits; }  // no empty split

  CUtensorMap tw, ta;
  if (!MakeMap(&tw, W, N, K, ldw, GEMM_BLOCK_N)) return -2;
  if (!MakeMap(&ta, A, M, K, lda, bt)) return -2;

  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.splits = splits; p.kb_per_split = kb_per; p.total_kb = total_kb;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.act_pair = act_pair;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.pdl = pdl_enabled;
  if (fused_ar) {
    if (device < 0 || device >= 16 || g_comm[device].world < 1 || !g_comm[device].buf[0]) return -2;
    const CommParams& c = g_comm[device];
    const long long n_out = act_pair ? N / 2 : N;
    // NVLS when the multicast buffers are registered and the launch fits their counters (ogb_comm_set_options: switch it
    // off, move the threshold between the one-shot and the two-shot form; the one-shot form pulls world * M * N * 2 bytes
    // out of every rank).
    const int nvls_env = ogb_comm_options()[0];
    const long long two_shot_bytes = ogb_comm_options()[1];
    const bool nvls = nvls_env && c.nv_data_mc && (long long)M * n_out <= c.nv_plane_elems &&
                      (long long)n_tiles * m_tiles * splits <= NV_MAX_CTAS && !(n_out % 8);
    if (n_out % 8 || (!nvls && (long long)M * n_out > c.plane_elems)) return -2;
    p.comm = c;
    p.comm_epilogue = 1;
    if (nvls) p.nvls = ((long long)c.world * M * n_out * 2 > two_shot_bytes && c.world > 2) ? 2 : 1;
    if (fused_rs) p.rs_rows = (M + c.world - 1) / c.world;
    else if (!nvls) {
      // one hop (every partial to every rank) costs world x the payload on the wire: fine for 2 ranks, not for 8
      const int two_shot = int(ogb_comm_options()[2]);
      if (two_shot == 1 || (two_shot == -1 && c.world >= 4)) p.ar2_rows = (M + c.world - 1) / c.world;
    }
  }
  if ((flags & 16) && fused_ar) return -1;   // the gathered form reads the previous call's epoch: it cannot open a call of its own
  if (flags & 16) {
    // all-gather -> GEMM: A is ignored; the activations come from the receive buffer filled by the previous fused call
    // (ogb_collective mode 3: every rank pushed its ceil(M / world) token rows of K values)
    if (device < 0 || device >= 16 || g_comm[device].world < 1 || !g_comm[device].buf[0]) return -2;
    const CommParams& c = g_comm[device];
    const int per = (M + c.world - 1) / c.world;
    if ((K % 8) || (long long)per * K > c.plane_elems) return -2;
    p.comm = c;          // the mainloop needs the buffer and epoch pointers; the epilogue stays local unless bits 2/3 are set
    p.ag_rows = per;
  }
  bool extras = false;
  if (f && f->norm_eps > 0.f) {
    if (p.ag_rows > 0) return -1;        // gathered activations are assembled by the warps that would sum the squares
    p.norm_eps = f->norm_eps;
    extras = true;
  }
  if (f && f->positions) {
    if (fused_ar || out_fp32 || act_pair || f->D <= 0 || (128 % f->D) || (f->rot % 16) || f->rot > f->D || N != (f->Hq + 2 * f->Hkv) * f->D ||
        !f->slots || !f->k_cache || !f->v_cache || (f->rot > 0 && (!f->cos || !f->sin)))
      return -1;
    p.rope.positions = f->positions; p.rope.slots = f->slots; p.rope.cos = f->cos; p.rope.sin = f->sin;
    p.rope.k_cache = static_cast<__nv_bfloat16*>(f->k_cache); p.rope.v_cache = static_cast<__nv_bfloat16*>(f->v_cache);
    p.rope.Hq = f->Hq; p.rope.Hkv = f->Hkv; p.rope.D = f->D; p.rope.rot = f->rot; p.rope.max_pos = f->max_pos;
    extras = true;
  }
  static const int persistent = [] { const char* e = getenv("OGB_GEMM_PERSISTENT"); return (e && e[0] == '0') ? 0 : 1; }();
  if (persistent && !extras && auto_split && bt == 256 && splits == 1 && !p.comm_epilogue && p.ag_rows == 0 && n_tiles * m_tiles >= sm_count)
    return LaunchPersistent(tw, ta, p, n_tiles, m_tiles, sm_count, stream);
  dim3 grid(n_tiles, m_tiles, splits);
  switch (bt) {
    case 16: return Launch<16>(tw, ta, p, grid, stream);
    case 32: return Launch<32>(tw, ta, p, grid, stream);
    case 64: return Launch<64>(tw, ta, p, grid, stream);
    case 128: return Launch<128>(tw, ta, p, grid, stream);
    case 256: return Launch<256>(tw, ta, p, grid, stream);
  }
  return -5;
}

// Grouped expert GEMM (mixture of experts): A holds `rows_total` token rows sorted by expert, W is
// [experts * N, K], the device-built tile list (ogb_moe_sort) gives for every token tile its expert, first
// row and row count.  C[row, :] = A[row, :] * W[expert(row)]^T (+ bias[expert]) (+ paired activation).
// `token_tile` must be the tile size the list was built for; `max_tiles` bounds the list length (the grid).
// flags bit 1: paired activation; act_kind selects it (1 = silu(gate)*up, 2 = clamped SwiGLU(alpha, limit)).
OGB_API int ogb_moe_gemm(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int rows_total, int N, int K, int experts,
                         const void* bias, int flags, int act_kind, float act_alpha, float act_limit, const int* tile_expert,
                         const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles, int token_tile,
                         int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows_total <= 0 || N <= 0 || K <= 0 || experts <= 0 || max_tiles <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  const int act_pair = (flags >> 1) & 1;
  if (act_pair && (N % 128)) return -1;
  if (max_tiles > 65535) return -1;
  static const int pdl_enabled = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  const int bt = token_tile;
  CUtensorMap tw, ta;
  if (!MakeMap(&tw, W, experts * N, K, ldw, GEMM_BLOCK_N)) return -2;
  if (!MakeMap(&ta, A, rows_total, K, lda, bt)) return -2;
  GemmParams p = {};
  p.M = rows_total; p.N = N; p.K = K;
  p.total_kb = (K + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  p.splits = 1; p.kb_per_split = p.total_kb;
  p.C = C; p.ldc = ldc; p.out_fp32 = flags & 1; p.act_pair = act_pair ? act_kind : 0;
  p.act_alpha = act_alpha; p.act_limit = act_limit;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.pdl = pdl_enabled;
  p.grp.tile_expert = tile_expert; p.grp.tile_row0 = tile_row0; p.grp.tile_rows = tile_rows; p.grp.num_tiles = num_tiles;
  dim3 grid((N + GEMM_BLOCK_N - 1) / GEMM_BLOCK_N, max_tiles, 1);
  switch (bt) {
    case 16: return Launch<16>(tw, ta, p, grid, stream);
    case 32: return Launch<32>(tw, ta, p, grid, stream);
    case 64: return Launch<64>(tw, ta, p, grid, stream);
    case 128: return Launch<128>(tw, ta, p, grid, stream);
    case 256: return Launch<256>(tw, ta, p, grid, stream);
  }
  return -5;
}
