// Shared pieces of the tcgen05 linear-layer kernels (bf16 weights in gemm_tcgen05.cu, int4 block-32
// weights in gemm_w4.cu): problem description, cluster / distributed-shared-memory / programmatic-launch /
// system-scope helpers, and the common epilogue: park the TMEM accumulator tile in shared memory,
// reduce the split-K cluster through distributed shared memory, apply bias / paired SiLU*mul / residual,
// store 16-byte row segments, or run the fused tensor-parallel all-reduce over NVLink peer memory.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace ogb {

constexpr int GEMM_BLOCK_N = 128;
constexpr int GEMM_BLOCK_K = 64;
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int W_TILE_BYTES = GEMM_BLOCK_N * GEMM_BLOCK_K * 2;  // 16 KiB
constexpr int COMM_MAX_WORLD = 8;

// Symmetric buffers of the fused all-reduce.  Payload travels in 16-byte lines {data, flag, data, flag}: eight bytes
// of data and the call's flag twice, written with one 16-byte peer store whose two halves are each atomic, so a
// reader that sees the expected flag in both halves has the data: no fence, no separate arrival flag, no barrier.
// All fused calls of a device form one sequence numbered by a device-side epoch (the same sequence on every rank): call
// e writes parity e & 1 of the receive buffers with flag e + 1.  A rank cannot start call e + 2 (which reuses the
// parity of call e) before it has finished call e + 1, i.e. before it has read every peer's lines of call e + 1, which
// those peers wrote after finishing call e: no second barrier, whatever the mapping of slices to CTAs.
struct CommParams {
  int world, rank;                        // world <= 1 with buf[0] == nullptr disables the fused all-reduce
  uint4* buf[COMM_MAX_WORLD];             // receive buffer of every rank: [2 parities][world sources][plane_elems / 4 lines]
  uint32_t* epoch;                        // this rank: [0] = calls finished so far, [1] = CTAs of the running call that are done
  long long plane_elems;                  // bf16 elements per source plane (4 per line)
  // NVLS (NVSwitch multicast) form of the same reductions; nv_data_mc == nullptr: not available, the flagged lines serve.
  // Every rank keeps its partial sums in its own `nv_data` plane (plain bf16, no flags); after a per-CTA arrival barrier
  // (one multimem.red on a counter that exists on every rank) a rank reads the SUM of all ranks' planes with
  // multimem.ld_reduce through the multicast mapping - the switch adds, fp32 accumulation.
  __nv_bfloat16* nv_data;                 // this rank: [2 parities][nv_plane_elems] partial sums
  __nv_bfloat16* nv_data_mc;              // the same range of every rank through the multicast mapping
  __nv_bfloat16* nv_out;                  // this rank: [2 parities][nv_plane_elems] sums broadcast by their owners (two-shot form)
  __nv_bfloat16* nv_out_mc;
  uint32_t* nv_ctr;                       // this rank: [2 phases][NV_MAX_CTAS] arrival counters, only ever incremented
  uint32_t* nv_ctr_mc;
  uint32_t* nv_expected;                  // this rank only (not symmetric): [2 phases][NV_MAX_CTAS] counter value after the last completed use
  long long nv_plane_elems;
};

constexpr int NV_MAX_CTAS = 4096;         // CTAs (or chunks) of one NVLS call; each has its own counter

// Registered symmetric buffers of a device (gemm_tcgen05.cu); nullptr when the index is out of range.
const CommParams* ogb_comm_params(int device);
// {use NVLS when registered, two-shot threshold in bytes}; see ogb_comm_set_options.
const long long* ogb_comm_options();

// Grouped (mixture-of-experts) mode: the token rows are sorted by expert and blockIdx.y walks a device-built
// list of token tiles, each inside one expert's row range; the weight is [experts * N, K].
struct GroupParams {
  const int* tile_expert;   // nullptr: not grouped
  const int* tile_row0;     // first (sorted) token row of the tile
  const int* tile_rows;     // rows of the tile that belong to its expert (<= token tile)
  const int* num_tiles;     // device scalar: tiles in use; CTAs beyond it return at once
};

// Rotary embedding + KV-cache append fused into the epilogue of a QKV projection (positions == nullptr: off).  Output
// columns are [Hq query heads | Hkv key heads | Hkv value heads] of D each; the rotation pairs element i with i + rot / 2
// (the non-interleaved form); keys and values go to row `slots[m]` of the caches [slots, Hkv, D] (slot < 0: nowhere).
struct FusedRope {
  const int* positions;
  const int* slots;
  const float* cos;     // [max_pos, rot / 2] fp32
  const float* sin;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int Hq, Hkv, D, rot, max_pos;
};

struct GemmParams {
  int M, N, K;          // N = weight rows (per expert when grouped)
  int splits, kb_per_split, total_kb;
  void* C;
  int ldc;
  int out_fp32;         // 0 bf16, 1 fp32, 2 fp16 output
  int act_pair;         // tiles hold 64 gate rows + 64 up rows, output has N/2 columns: 1 = silu(gate)*up,
                        // 2 = clamped SwiGLU: g = min(gate, limit), u = clamp(up, +-limit), g*sigmoid(alpha*g)*(u+1)
  float act_alpha, act_limit;
  const __nv_bfloat16* residual;
  int ldr;
  const __nv_bfloat16* bias;
  int* status;
  int pdl;
  CommParams comm;
  int comm_epilogue;    // 1: the epilogue runs the fused all-reduce / reduce-scatter (and the call closes an epoch)
  int ag_rows;          // > 0: all-gather -> GEMM: the activations are not read through the tensor map but assembled from the
                        // flagged lines that the ranks pushed into this rank's receive buffer in the previous fused call
                        // (rank r pushed token rows [r * ag_rows, (r + 1) * ag_rows) as [row][K] into its plane)
  int ar2_rows;         // > 0: the all-reduce runs in two hops (reduce-scatter by token rows to an owner rank, which sums and
                        // broadcasts): each partial crosses NVLink once instead of world times; owner of row m = m / ar2_rows
  int rs_rows;          // > 0: reduce-scatter by token rows: rank r receives (and stores, as its rows 0..) rows [r * rs_rows, (r + 1) * rs_rows)
  int nvls;             // comm_epilogue through NVSwitch multicast: 1 = one-shot (every rank reads the sum of its whole slice with
                        // multimem.ld_reduce), 2 = two-shot (a rank reduces 1/world of the slice and multicasts the sums)
  GroupParams grp;
  float norm_eps;       // > 0: RMS norm folded into this GEMM - the activations are the un-normalised rows, the weight carries the
                        // norm's weight, the kernel sums the squares of each row as its tiles pass through shared memory and the
                        // epilogue multiplies row m by rsqrt(mean(x_m^2) + eps)
  FusedRope rope;
};

// DEEP: one CTA per SM with a pipeline twice as deep, for launches of at most one CTA per SM (the same bytes in flight per SM
// as two resident CTAs of the shallow form would have, which such a launch never gets).
template <int BT, bool DEEP = false>
struct GemmCfg {
  static constexpr int A_TILE_BYTES = BT * GEMM_BLOCK_K * 2;
  static constexpr int STAGE_BYTES = W_TILE_BYTES + A_TILE_BYTES;
  // Decode-sized tiles keep two CTAs per SM: more bytes in flight per SM, dynamic balance between
  // SMs, and room for the next kernel's CTAs to become resident and prefetch weights.
  static constexpr bool TWO_PER_SM = BT <= 128 && !DEEP;   // 128-token tiles: two CTAs per SM, one's epilogue under the other's main loop
  static constexpr int BUDGET = TWO_PER_SM ? 100 * 1024 : 196 * 1024;
  static constexpr int MAX_STAGES = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > (DEEP ? 12 : 8) ? (DEEP ? 12 : 8) : MAX_STAGES;
  static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  static constexpr int PARTIAL_BYTES = BT * GEMM_BLOCK_N * 4;  // fp32 tile parked in stage memory
  static constexpr int SSQ_OFFSET = STAGES * STAGE_BYTES + 512;   // per-row sums of squares (folded norm), after the barriers
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/ + BT * 4;
  static_assert(PARTIAL_BYTES + 16 * 128 * 16 <= STAGES * STAGE_BYTES, "the parked tile and the reduction's staging lines must fit in the pipeline memory");
};

__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t comm_flag(uint32_t epoch) { const uint32_t f = epoch + 1u; return f ? f : 1u; }
// One line: 8 bytes of data + the flag in both halves (each 8-byte half of the store is atomic).
__device__ __forceinline__ void st_line(uint4* p, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Waits (bounded) for a line of this call.  `dead` is the thread's give-up state: set when the device already carries a
// failed wait or when this wait runs out (the status word is updated), after which lines are taken as they are.
__device__ __forceinline__ uint4 wait_line(const uint4* p, uint32_t flag, bool& dead, int* status) {
  uint4 v = ld_line(p);
  if (v.y == flag && v.w == flag) return v;
  if (dead) return v;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    v = ld_line(p);
    if (v.y == flag && v.w == flag) return v;
    if ((++spins & 0x3f) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0 || global_timer_ns() - t0 > 2000000000ull) {
        atomicMax(status, OGB_ERR_WAIT_PEER);
        dead = true;
        return v;
      }
    }
  }
}

// ------------------------------------------------------------------------------- NVLS (multimem) helpers
// Sum over all ranks of eight bf16 values at the same offset of every rank's buffer (fp32 accumulation in the switch).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
// One 16-byte store that lands at the same offset of every rank's buffer.
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
// Adds 1 to the counter at the same offset on every rank; the release makes this CTA's earlier stores (ordered before it by a
// CTA barrier) visible to whoever acquires the counter.
__device__ __forceinline__ void multimem_signal(uint32_t* mc_ctr) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ctr), "r"(1u) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Arrival barrier between the CTAs with index `slot` of every rank, run by ONE thread: announce this rank, then wait
// (bounded) until all `world` ranks have.  Counters only grow; the local `expected` word remembers the value the last use
// ended on, so nothing is ever reset and the sequence replays inside CUDA graphs.  Returns false when the wait ran out.
__device__ __forceinline__ bool nvls_arrive_and_wait(const CommParams& c, int phase, unsigned slot, int* status) {
  uint32_t* exp = c.nv_expected + phase * NV_MAX_CTAS + slot;
  const uint32_t target = *exp + uint32_t(c.world);
  *exp = target;
  multimem_signal(c.nv_ctr_mc + phase * NV_MAX_CTAS + slot);
  const uint32_t* mine = c.nv_ctr + phase * NV_MAX_CTAS + slot;
  if (int32_t(ld_acquire_sys_u32(mine) - target) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (int32_t(ld_acquire_sys_u32(mine) - target) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0 || global_timer_ns() - t0 > 2000000000ull) {
        atomicMax(status, OGB_ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

// Opens a fused call for this CTA, run by ONE thread after the kernel's dependency wait (the previous call of the device has
// completed): returns the call's epoch and counts the CTA; the last CTA of the grid to get here publishes epoch + 1 for the
// next call.  Nothing of this call depends on that store (the next call reads the epoch only after this grid has completed),
// so the bookkeeping sits at the start of the kernel, under the main loop, instead of on the tail every CTA must finish.
__device__ __forceinline__ uint32_t comm_open_call(const CommParams& c, unsigned total_ctas) {
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(c.epoch);
  __threadfence();                       // the read above is performed before this CTA is counted
  if (atomicAdd(c.epoch + 1, 1u) == total_ctas - 1) {
    c.epoch[1] = 0;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(c.epoch) = e + 1;
  }
  return e;
}

// Output side of the epilogue, kept out of line: the epilogue runs once per CTA, so its instructions are fetched cold, and
// every inlined copy of this routine (three output types, vector and tail forms) costs instruction-cache misses.
struct StoreArgs {
  void* C;
  const __nv_bfloat16* residual;
  int ldc, ldr, out_kind, n_out;    // out_kind: 0 bf16, 1 fp32, 2 fp16
};
static __device__ __noinline__ void epi_store8(const StoreArgs a, int m, int col, float4 lo, float4 hi) {
  float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  const bool full = col + 8 <= a.n_out;
  if (a.residual) {
    const __nv_bfloat16* r = a.residual + size_t(m) * a.ldr + col;
    if (full && (reinterpret_cast<uintptr_t>(r) & 15) == 0) {
      const uint4 q = *reinterpret_cast<const uint4*>(r);
      const float2 x0 = unpack_bf16x2(q.x), x1 = unpack_bf16x2(q.y), x2 = unpack_bf16x2(q.z), x3 = unpack_bf16x2(q.w);
      v[0] += x0.x; v[1] += x0.y; v[2] += x1.x; v[3] += x1.y; v[4] += x2.x; v[5] += x2.y; v[6] += x3.x; v[7] += x3.y;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (col + j < a.n_out) v[j] += bf2f(r[j]);
    }
  }
  if (a.out_kind == 1) {
    float* dst = reinterpret_cast<float*>(a.C) + size_t(m) * a.ldc + col;
    if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (col + j < a.n_out) dst[j] = v[j];
    }
  } else if (a.out_kind == 2) {   // fp16 output (feeds the fp16 form of the packed FP4 expert GEMM)
    __half* dst = reinterpret_cast<__half*>(a.C) + size_t(m) * a.ldc + col;
    if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]), pack_f16x2(v[6], v[7]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (col + j < a.n_out) dst[j] = __float2half_rn(v[j]);
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.C) + size_t(m) * a.ldc + col;
    if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (col + j < a.n_out) dst[j] = f2bf(v[j]);
    }
  }
}

// Epilogue shared by the linear-layer kernels.  Called by all threads of the CTA once the MMA issuer has committed the last
// k-block to `accum_bar`; `smem` is the (idle) pipeline memory, reused for the fp32 tile.
// COMM: 0 = results stay on this GPU; 1 = tensor-parallel reduction with flagged lines over peer memory; 2 = through the
// NVSwitch multicast mapping (NVLS).  A template parameter because the epilogue's instructions are fetched cold once per
// CTA: the local form must not carry the reductions' code.
// ssq: shared-memory array of the per-token-row sums of squares of this CTA's share of the activations (norm folded into the
// GEMM, p.norm_eps > 0), or nullptr.
template <int BT, int COMM>
__device__ __forceinline__ void gemm_epilogue(const GemmParams& p, uint8_t* smem, uint32_t tmem_base, uint64_t* accum_bar,
                                              volatile int* abort_flag, volatile uint32_t* use_slot, int n_tile, int m_tile,
                                              int row0, int rows, int bias_off, const float* ssq = nullptr, int n_acc = 1) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto fail = [&](int code) { atomicMax(p.status, code); *abort_flag = 1; };
  // -------------------------------------------------------------------- epilogue (warps 2..5)
  const bool epi = warp >= 2 && warp < 6;   // kernels with more than six warps: the others only meet the CTA-wide barriers
  const int et = threadIdx.x - 64;   // 0..127 for epilogue threads
  float* part = reinterpret_cast<float*>(smem);  // [BT][128] fp32, reuses the pipeline stages
  if (epi) {
    const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
    const int row = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
    if (!mbar_wait_bounded(accum_bar, 0, abort_flag, 4000000000ull)) fail(OGB_ERR_WAIT_MMA);
    asm volatile("bar.sync 1, 128;" ::: "memory");  // uniform decision over the 128 epilogue threads
    const bool have = (*abort_flag == 0);
    tc_fence_after();
    if (have) {
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 16) {
        uint32_t r0[16];
        tmem_ld16(taddr + c0, r0);
        tmem_ld_wait();
        // n_acc > 1 (packed FP4 experts): the k-steps went round-robin into n_acc accumulators BT columns apart; sum them
        for (int a = 1; a < n_acc; ++a) {
          uint32_t r1[16];
          tmem_ld16(taddr + a * BT + c0, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) r0[j] = __float_as_uint(__uint_as_float(r0[j]) + __uint_as_float(r1[j]));
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) part[(c0 + j) * GEMM_BLOCK_N + row] = __uint_as_float(r0[j]);
      }
    }
    if (p.pdl) pdl_wait();  // residual reads and every store come after the previous kernel has finished
  }
  // The parked tiles are complete and visible (cluster-wide when split) after this barrier.  Every
  // thread of every CTA of the cluster meets here, also after an abort.
  __syncwarp();
  if (p.splits > 1) cluster_sync_all(); else __syncthreads();

  if (epi && *abort_flag == 0) {
    const int my_rank = p.splits > 1 ? int(cluster_ctarank()) : 0;
    const int per = (BT + p.splits - 1) / p.splits;  // token columns finished by this CTA
    const int c_begin = min(BT, my_rank * per), c_end = min(BT, c_begin + per);
    const int OCT = p.act_pair ? 8 : 16;             // 8-wide output segments per token column
    const int items = (c_end - c_begin) * OCT;
    const int n_out = p.act_pair ? p.N / 2 : p.N;    // output columns of the whole problem
    const int col0 = n_tile * (p.act_pair ? 64 : 128);
    const uint32_t part_addr = smem_u32(part);
    const StoreArgs sa{p.C, p.residual, p.ldc, p.ldr, p.out_fp32, n_out};

    // sum over the split-K cluster of 8 accumulators of token column mc, weight rows n_local.., scaled by the folded norm
    auto reduce8 = [&](int mc, int n_local, float scale, float (&v)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      for (int s = 0; s < p.splits; ++s) {
        float4 a, b;
        if (p.splits > 1) {
          const uint32_t ra = dsmem_addr(part_addr + uint32_t(mc * GEMM_BLOCK_N + n_local) * 4, uint32_t(s));
          a = ld_dsmem_f32x4(ra);
          b = ld_dsmem_f32x4(ra + 16);
        } else {
          a = *reinterpret_cast<const float4*>(part + mc * GEMM_BLOCK_N + n_local);
          b = *reinterpret_cast<const float4*>(part + mc * GEMM_BLOCK_N + n_local + 4);
        }
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
      const int n_glob = n_tile * GEMM_BLOCK_N + n_local;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[j] *= scale;
        if (p.bias && n_glob + j < p.N) v[j] += bf2f(p.bias[bias_off + n_glob + j]);
      }
    };
    // 1 / rms of token column mc's activation row (norm folded into this GEMM: the weight already carries the norm's weight)
    auto row_scale = [&](int mc) {
      if (ssq == nullptr) return 1.f;
      float t = 0.f;
      if (p.splits > 1) {
        for (int s = 0; s < p.splits; ++s) {
          float x;
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(x) : "r"(dsmem_addr(smem_u32(ssq + mc), uint32_t(s))) : "memory");
          t += x;
        }
      } else {
        t = ssq[mc];
      }
      return rsqrtf(t / float(p.K) + p.norm_eps);
    };

    // Epoch of this call: read (and the call counted) by the kernel's producer thread right after its dependency wait, long
    // before the epilogue (comm_open_call); visible here through the CTA-wide barrier above.
    const uint32_t use = COMM != 0 ? *use_slot : 0u;
    const uint32_t flag = comm_flag(use);
    const size_t plane_lines = size_t(p.comm.plane_elems) / 4;
    const size_t par_off = size_t(use & 1) * p.comm.world * plane_lines;

#pragma unroll 1
    for (int item = et; item < items; item += 128) {
      const int mc = c_begin + item / OCT, oc = item % OCT;
      const int m = row0 + mc;
      if (mc >= rows) continue;
      const float rs = row_scale(mc);
      float v[8];
      const int col = col0 + oc * 8;
      if (p.act_pair) {
        float u[8];
        reduce8(mc, oc * 8, rs, v);
        reduce8(mc, 64 + oc * 8, rs, u);
        if (p.act_pair == 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = silu(v[j]) * u[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g = p.act_limit > 0.f ? fminf(v[j], p.act_limit) : v[j];
            const float w = p.act_limit > 0.f ? fminf(fmaxf(u[j], -p.act_limit), p.act_limit) : u[j];
            v[j] = g / (1.f + __expf(-p.act_alpha * g)) * (w + 1.f);
          }
        }
      } else {
        const bool roped = COMM == 0 && p.rope.positions != nullptr;
        // the token's position and cache slot are fetched first: their latency passes under the reduction below
        const int pos_raw = roped ? p.rope.positions[m] : 0;
        const int slot = roped ? p.rope.slots[m] : -1;
        reduce8(mc, oc * 8, rs, v);
        if (roped) {
          // Fused rotary embedding + KV-cache append of a QKV projection (heads never straddle a tile: 128 % D == 0).
          // Query heads go to C rotated; key heads go rotated, value heads as they are, to this token's cache slot.
          const FusedRope& R = p.rope;
          const int head = col / R.D, d = col - head * R.D;
          if (head < R.Hq + R.Hkv && d < R.rot) {
            const int half = R.rot >> 1;
            const bool first = d < half;
            const int pos = pos_raw < 0 ? 0 : (pos_raw >= R.max_pos ? R.max_pos - 1 : pos_raw);
            const size_t ci = size_t(pos) * half + (first ? d : d - half);      // a multiple of 8: 32-byte aligned rows of 8 floats
            const float4 c0 = *reinterpret_cast<const float4*>(R.cos + ci), c1 = *reinterpret_cast<const float4*>(R.cos + ci + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(R.sin + ci), s1 = *reinterpret_cast<const float4*>(R.sin + ci + 4);
            float u[8];
            reduce8(mc, first ? oc * 8 + half : oc * 8 - half, rs, u);
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = first ? v[j] * cs[j] - u[j] * sn[j] : v[j] * cs[j] + u[j] * sn[j];
          }
          if (head >= R.Hq) {
            if (slot >= 0 && col < p.N) {
              const bool is_k = head < R.Hq + R.Hkv;
              __nv_bfloat16* dst = (is_k ? R.k_cache : R.v_cache) + (size_t(slot) * R.Hkv + (head - R.Hq - (is_k ? 0 : R.Hkv))) * R.D + d;
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
            }
            continue;
          }
        }
      }
      if (COMM == 0) {
        epi_store8(sa, m, col, make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]));
      } else if (COMM == 2) {
        // this rank's partial stays in its own plane; the switch adds the planes when a rank reads through the multicast mapping
        if (col < n_out)
          *reinterpret_cast<uint4*>(p.comm.nv_data + size_t(use & 1) * p.comm.nv_plane_elems + size_t(m) * n_out + col) =
              make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
      } else if (col < n_out) {
        // push this rank's partial (bf16) into every rank's receive buffer (all-reduce) or into the buffer of the rank
        // that owns the token row (reduce-scatter, two-hop all-reduce): two flagged lines per 8 values
        const size_t line = par_off + size_t(p.comm.rank) * plane_lines + (size_t(m) * n_out + col) / 4;
        const uint32_t d0 = pack_bf16x2(v[0], v[1]), d1 = pack_bf16x2(v[2], v[3]), d2 = pack_bf16x2(v[4], v[5]), d3 = pack_bf16x2(v[6], v[7]);
        const int own_rows = p.rs_rows > 0 ? p.rs_rows : p.ar2_rows;      // > 0: the partial goes to the row's owner only
        const int r_lo = own_rows > 0 ? m / own_rows : 0, r_hi = own_rows > 0 ? r_lo + 1 : p.comm.world;
        for (int r = r_lo; r < r_hi; ++r) {
          st_line(p.comm.buf[r] + line, d0, d1, flag);
          st_line(p.comm.buf[r] + line + 1, d2, d3, flag);
        }
      }
    }

    auto unpack8 = [&](const uint4& q, float (&w)[8]) {
      const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y; w[4] = c.x; w[5] = c.y; w[6] = d.x; w[7] = d.y;
    };
    if (COMM == 2) {
      // ---- NVLS: barrier with the same CTA of every rank, then read sums through the switch.
      const unsigned slot = (blockIdx.y * gridDim.x + blockIdx.x) * gridDim.z + blockIdx.z;   // the grid is the same on every rank
      const size_t par = size_t(use & 1) * p.comm.nv_plane_elems;
      auto rank_barrier = [&](int phase) {
        asm volatile("bar.sync 1, 128;" ::: "memory");   // every thread's stores of this phase are ordered before thread 0's release
        if (et == 0 && *abort_flag == 0 && !nvls_arrive_and_wait(p.comm, phase, slot, p.status)) *abort_flag = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        return *abort_flag == 0;
      };
      if (rank_barrier(0)) {
        const bool one_shot = p.nvls == 1 || p.rs_rows > 0;
        // one-shot: the sum of every item of the slice (reduce-scatter: of the rows this rank keeps).
        // two-shot: each rank reduces every world-th item and multicasts the sum into every rank's `nv_out` plane; after a
        // second barrier all sums of the slice are local.  A partial crosses NVLink once, a sum once.
        int j = 0;
#pragma unroll 1
        for (int item = et; item < items; item += 128, ++j) {
          const int mc = c_begin + item / OCT, oc = item % OCT;
          const int m = row0 + mc, col = col0 + oc * 8;
          if (mc >= rows || col >= n_out) continue;
          const size_t off = par + size_t(m) * n_out + col;
          if (one_shot) {
            if (p.rs_rows > 0 && m / p.rs_rows != p.comm.rank) continue;
            float w[8];
            unpack8(multimem_ld_reduce_bf16x8(p.comm.nv_data_mc + off), w);
            epi_store8(sa, p.rs_rows > 0 ? m - p.comm.rank * p.rs_rows : m, col, make_float4(w[0], w[1], w[2], w[3]), make_float4(w[4], w[5], w[6], w[7]));
          } else if ((j + et) % p.comm.world == p.comm.rank) {
            multimem_st_b128(p.comm.nv_out_mc + off, multimem_ld_reduce_bf16x8(p.comm.nv_data_mc + off));
          }
        }
        if (!one_shot && rank_barrier(1)) {
#pragma unroll 1
          for (int item = et; item < items; item += 128) {
            const int mc = c_begin + item / OCT, oc = item % OCT;
            const int m = row0 + mc, col = col0 + oc * 8;
            if (mc >= rows || col >= n_out) continue;
            float w[8];
            unpack8(ld_line(reinterpret_cast<const uint4*>(p.comm.nv_out + par + size_t(m) * n_out + col)), w);
            epi_store8(sa, m, col, make_float4(w[0], w[1], w[2], w[3]), make_float4(w[4], w[5], w[6], w[7]));
          }
        }
      }
    } else if (COMM == 1) {
      // Every thread collects the lines of the items it pushed itself: its own pushes are long under way, and the peers'
      // lines of the same items arrive at about the same time.  The data carries its own arrival flag.
      // A thread's lines are fetched sixteen at a time by asynchronous copies (L2 -> shared memory, all in flight together: a
      // chain of dependent loads would cost one L2 round trip per line) into staging slots behind the parked tile; only
      // lines that had not arrived yet are then waited for one by one.  Short loops on purpose: this code is fetched cold.
      bool dead = false;      // the waits themselves look at the status word from time to time
      const int W = p.comm.world;
      const uint4* my_buf = p.comm.buf[p.comm.rank] + par_off;
      uint4* stage = reinterpret_cast<uint4*>(smem + GemmCfg<BT>::PARTIAL_BYTES);   // [16 slots][128 threads] lines
      // The reductions never pair columns (OCT == 16): thread et owns segment et % 16 of token columns c_begin + et / 16 + 8 k.
      const int seg_col = col0 + (et & 15) * 8;
      const int mc_first = c_begin + (et >> 4), mc_end = min(c_end, rows);
      const size_t row_lines = size_t(n_out) / 4;
      // hop: 0 = one-hop all-reduce / reduce-scatter (sum the W planes of the rows kept here), 1 = two-hop, owner's part (sum
      // the W planes of the owned rows, store, broadcast), 2 = two-hop, the other rows (one plane: the owner's sums)
#pragma unroll 1
      for (int hop = (p.ar2_rows > 0 ? 1 : 0); hop <= (p.ar2_rows > 0 ? 2 : 0); ++hop) {
        const int per_item = hop == 2 ? 2 : 2 * W;
        // walk (item, line of the item) pairs: `mc` is the item's token column, `rem` the line (plane * 2 + half)
        int mc = mc_first, rem = 0;
        auto item_ok = [&](int mc_) {      // is this token column collected in this hop?
          const int m = row0 + mc_;
          if (hop == 0) return p.rs_rows == 0 || m / p.rs_rows == p.comm.rank;
          return (m / p.ar2_rows == p.comm.rank) == (hop == 1);
        };
        while (mc < mc_end && !item_ok(mc)) mc += 8;
        float v[8];
        auto line_ptr = [&](int mc_, int rem_) {
          const int m = row0 + mc_;
          const int plane = hop == 2 ? m / p.ar2_rows : (rem_ >> 1);
          return my_buf + size_t(plane) * plane_lines + size_t(m) * row_lines + (seg_col >> 2) + (rem_ & 1);
        };
        auto advance = [&](int& mc_, int& rem_) {
          if (++rem_ < per_item) return;
          rem_ = 0;
          mc_ += 8;
          while (mc_ < mc_end && !item_ok(mc_)) mc_ += 8;
        };
#pragma unroll 1
        while (mc < mc_end && seg_col < n_out) {
          // pass 1: asynchronous copies of up to 16 lines into this thread's staging slots (all in flight together)
          int mc_w = mc, rem_w = rem, n = 0;
#pragma unroll 1
          for (; n < 16 && mc_w < mc_end; ++n) {
            cp_async16(stage + (n * 128 + et), line_ptr(mc_w, rem_w), true);
            advance(mc_w, rem_w);
          }
          cp_async_commit();
          cp_async_wait<0>();
          // pass 2: the same walk; a line whose flag is not this call's had not arrived yet and is waited for in place
#pragma unroll 1
          for (int i = 0; i < n; ++i) {
            uint4 q = stage[i * 128 + et];
            if (q.y != flag || q.w != flag) q = wait_line(line_ptr(mc, rem), flag, dead, p.status);
            const int h4 = (rem & 1) * 4;
            const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.z);
            if (rem < 2) { v[h4] = a.x; v[h4 + 1] = a.y; v[h4 + 2] = b.x; v[h4 + 3] = b.y; }
            else { v[h4] += a.x; v[h4 + 1] += a.y; v[h4 + 2] += b.x; v[h4 + 3] += b.y; }
            if (rem == per_item - 1) {
              const int m = row0 + mc;
              if (hop == 1) {
                // the owner rounds to bf16 (every rank ends up with the same bits) and broadcasts the sums as flagged lines
                // into plane `owner` of every other rank - a plane position no hop-1 line of this call uses there
                const size_t line = par_off + size_t(p.comm.rank) * plane_lines + size_t(m) * row_lines + (seg_col >> 2);
                const uint32_t d0 = pack_bf16x2(v[0], v[1]), d1 = pack_bf16x2(v[2], v[3]), d2 = pack_bf16x2(v[4], v[5]), d3 = pack_bf16x2(v[6], v[7]);
                for (int r = 0; r < W; ++r) {
                  if (r == p.comm.rank) continue;
                  st_line(p.comm.buf[r] + line, d0, d1, flag);
                  st_line(p.comm.buf[r] + line + 1, d2, d3, flag);
                }
                unpack8(make_uint4(d0, d1, d2, d3), v);
              }
              epi_store8(sa, p.rs_rows > 0 ? m - p.comm.rank * p.rs_rows : m, seg_col, make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]));
            }
            advance(mc, rem);
          }
        }
      }
      if (dead) *abort_flag = 1;
    }
  }
  if (p.splits > 1) {
    __syncwarp();
    cluster_sync_all();  // no CTA leaves while a peer may still read its shared memory
  }
}

}  // namespace ogb
