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
};

// Registered symmetric buffers of a device (gemm_tcgen05.cu); nullptr when the index is out of range.
const CommParams* ogb_comm_params(int device);

// Grouped (mixture-of-experts) mode: the token rows are sorted by expert and blockIdx.y walks a device-built
// list of token tiles, each inside one expert's row range; the weight is [experts * N, K].
struct GroupParams {
  const int* tile_expert;   // nullptr: not grouped
  const int* tile_row0;     // first (sorted) token row of the tile
  const int* tile_rows;     // rows of the tile that belong to its expert (<= token tile)
  const int* num_tiles;     // device scalar: tiles in use; CTAs beyond it return at once
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
  GroupParams grp;
};

template <int BT>
struct GemmCfg {
  static constexpr int A_TILE_BYTES = BT * GEMM_BLOCK_K * 2;
  static constexpr int STAGE_BYTES = W_TILE_BYTES + A_TILE_BYTES;
  // Decode-sized tiles keep two CTAs per SM: more bytes in flight per SM, dynamic balance between
  // SMs, and room for the next kernel's CTAs to become resident and prefetch weights.
  static constexpr bool TWO_PER_SM = BT <= 128;   // 128-token tiles: two CTAs per SM, one's epilogue under the other's main loop
  static constexpr int BUDGET = TWO_PER_SM ? 100 * 1024 : 196 * 1024;
  static constexpr int MAX_STAGES = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
  static constexpr int PARTIAL_BYTES = BT * GEMM_BLOCK_N * 4;  // fp32 tile parked in stage memory
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(PARTIAL_BYTES <= STAGES * STAGE_BYTES, "the parked tile must fit in the pipeline memory");
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

// Epilogue shared by the linear-layer kernels.  Called by all 192 threads of the CTA once the MMA issuer has
// committed the last k-block to `accum_bar`; `smem` is the (idle) pipeline memory, reused for the fp32 tile.
template <int BT>
__device__ __forceinline__ void gemm_epilogue(const GemmParams& p, uint8_t* smem, uint32_t tmem_base, uint64_t* accum_bar,
                                              volatile int* abort_flag, volatile uint32_t* use_slot, int n_tile, int m_tile,
                                              int row0, int rows, int bias_off, int n_acc = 1) {
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
    const bool comm_on = p.comm_epilogue != 0;

    auto reduce8 = [&](int mc, int n_local, float (&v)[8]) {
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
    };
    auto add_bias8 = [&](int n_glob, float (&v)[8]) {
      if (!p.bias) return;
#pragma unroll
      for (int j = 0; j < 8; ++j) if (n_glob + j < p.N) v[j] += bf2f(p.bias[bias_off + n_glob + j]);
    };
    auto store8 = [&](int m, int col, float (&v)[8]) {  // residual add + store of one 8-wide segment
      if (p.residual) {
#pragma unroll
        for (int j = 0; j < 8; ++j) if (col + j < n_out) v[j] += bf2f(p.residual[size_t(m) * p.ldr + col + j]);
      }
      if (p.out_fp32 == 1) {
        float* dst = reinterpret_cast<float*>(p.C) + size_t(m) * p.ldc + col;
        if (col + 8 <= n_out && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (col + j < n_out) dst[j] = v[j];
        }
      } else if (p.out_fp32 == 2) {   // fp16 output (feeds the fp16 form of the packed FP4 expert GEMM)
        __half* dst = reinterpret_cast<__half*>(p.C) + size_t(m) * p.ldc + col;
        if (col + 8 <= n_out && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]), pack_f16x2(v[6], v[7]));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (col + j < n_out) dst[j] = __float2half_rn(v[j]);
        }
      } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(m) * p.ldc + col;
        if (col + 8 <= n_out && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (col + j < n_out) dst[j] = f2bf(v[j]);
        }
      }
    };

    uint32_t use = 0;   // epoch of this call
    if (comm_on) {
      // read after griddepcontrol.wait: the previous call has finished and published its increment
      if (et == 0) *use_slot = *reinterpret_cast<volatile uint32_t*>(p.comm.epoch);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      use = *use_slot;
    }
    const uint32_t flag = comm_flag(use);
    const size_t plane_lines = size_t(p.comm.plane_elems) / 4;
    const size_t par_off = size_t(use & 1) * p.comm.world * plane_lines;

    for (int item = et; item < items; item += 128) {
      const int mc = c_begin + item / OCT, oc = item % OCT;
      const int m = row0 + mc;
      if (mc >= rows) continue;
      float v[8];
      if (p.act_pair) {
        float u[8];
        reduce8(mc, oc * 8, v);
        reduce8(mc, 64 + oc * 8, u);
        add_bias8(n_tile * GEMM_BLOCK_N + oc * 8, v);
        add_bias8(n_tile * GEMM_BLOCK_N + 64 + oc * 8, u);
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
        reduce8(mc, oc * 8, v);
        add_bias8(n_tile * GEMM_BLOCK_N + oc * 8, v);
      }
      const int col = col0 + oc * 8;
      if (!comm_on) {
        store8(m, col, v);
      } else if (col < n_out) {
        // push this rank's partial (bf16) into every rank's receive buffer (all-reduce) or into the buffer of the rank
        // that owns the token row (reduce-scatter): two flagged lines per 8 values
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

    if (comm_on) {
      // Every thread collects the lines of the items it pushed itself: its own pushes are long under way, and the peers'
      // lines of the same items arrive at about the same time.  The data carries its own arrival flag.
      bool dead = *reinterpret_cast<volatile int*>(p.status) != 0;
      if (p.ar2_rows > 0) {
        // Two-hop all-reduce.  Hop 1 (above) sent every partial to the owner of its token row.  Here the owner sums the
        // world's partials of its rows in rank order, rounds to bf16 (so that every rank ends up with the same bits),
        // stores, and broadcasts the sums as flagged lines into plane `owner` of every other rank — a plane position no
        // hop-1 line of this call uses there; the other ranks then collect the rows they do not own.
        for (int item = et; item < items; item += 128) {
          const int mc = c_begin + item / OCT, oc = item % OCT;
          const int m = row0 + mc;
          const int col = col0 + oc * 8;
          if (mc >= rows || col >= n_out || m / p.ar2_rows != p.comm.rank) continue;
          float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          const size_t line = par_off + (size_t(m) * n_out + col) / 4;
          for (int r = 0; r < p.comm.world; ++r) {
            const uint4 q0 = wait_line(p.comm.buf[p.comm.rank] + line + size_t(r) * plane_lines, flag, dead, p.status);
            const uint4 q1 = wait_line(p.comm.buf[p.comm.rank] + line + size_t(r) * plane_lines + 1, flag, dead, p.status);
            const float2 a = unpack_bf16x2(q0.x), b = unpack_bf16x2(q0.z), c = unpack_bf16x2(q1.x), d = unpack_bf16x2(q1.z);
            v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
          }
          const uint32_t d0 = pack_bf16x2(v[0], v[1]), d1 = pack_bf16x2(v[2], v[3]), d2 = pack_bf16x2(v[4], v[5]), d3 = pack_bf16x2(v[6], v[7]);
          for (int r = 0; r < p.comm.world; ++r) {
            if (r == p.comm.rank) continue;
            st_line(p.comm.buf[r] + line + size_t(p.comm.rank) * plane_lines, d0, d1, flag);
            st_line(p.comm.buf[r] + line + size_t(p.comm.rank) * plane_lines + 1, d2, d3, flag);
          }
          const float2 a = unpack_bf16x2(d0), b = unpack_bf16x2(d1), c = unpack_bf16x2(d2), d = unpack_bf16x2(d3);
          float w[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
          store8(m, col, w);
        }
        for (int item = et; item < items; item += 128) {
          const int mc = c_begin + item / OCT, oc = item % OCT;
          const int m = row0 + mc;
          const int col = col0 + oc * 8;
          if (mc >= rows || col >= n_out) continue;
          const int owner = m / p.ar2_rows;
          if (owner == p.comm.rank) continue;
          const uint4* src = p.comm.buf[p.comm.rank] + par_off + size_t(owner) * plane_lines + (size_t(m) * n_out + col) / 4;
          const uint4 q0 = wait_line(src, flag, dead, p.status);
          const uint4 q1 = wait_line(src + 1, flag, dead, p.status);
          const float2 a = unpack_bf16x2(q0.x), b = unpack_bf16x2(q0.z), c = unpack_bf16x2(q1.x), d = unpack_bf16x2(q1.z);
          float w[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
          store8(m, col, w);
        }
      }
      for (int item = et; item < items && p.ar2_rows == 0; item += 128) {
        const int mc = c_begin + item / OCT, oc = item % OCT;
        const int m = row0 + mc;
        const int col = col0 + oc * 8;
        if (mc >= rows || col >= n_out) continue;
        if (p.rs_rows > 0 && m / p.rs_rows != p.comm.rank) continue;   // another rank's row
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const uint4* base = p.comm.buf[p.comm.rank] + par_off + (size_t(m) * n_out + col) / 4;
        for (int r = 0; r < p.comm.world; ++r) {   // rank order: bit-identical sums on every rank
          const uint4 q0 = wait_line(base + size_t(r) * plane_lines, flag, dead, p.status);
          const uint4 q1 = wait_line(base + size_t(r) * plane_lines + 1, flag, dead, p.status);
          const float2 a = unpack_bf16x2(q0.x), b = unpack_bf16x2(q0.z), c = unpack_bf16x2(q1.x), d = unpack_bf16x2(q1.z);
          v[0] += a.x; v[1] += a.y; v[2] += b.x; v[3] += b.y; v[4] += c.x; v[5] += c.y; v[6] += d.x; v[7] += d.y;
        }
        store8(p.rs_rows > 0 ? m - p.comm.rank * p.rs_rows : m, col, v);
      }
      if (dead) *abort_flag = 1;
    }
  }
  if (p.splits > 1) {
    __syncwarp();
    cluster_sync_all();  // no CTA leaves while a peer may still read its shared memory
  }
  if (p.comm_epilogue) {
    // The last CTA of the call to get here closes the epoch (every CTA passes this point, also after an abort).
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned total = gridDim.x * gridDim.y * gridDim.z;
      if (atomicAdd(p.comm.epoch + 1, 1u) == total - 1) {
        p.comm.epoch[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.comm.epoch) = *reinterpret_cast<volatile uint32_t*>(p.comm.epoch) + 1;
      }
    }
  }

}

}  // namespace ogb
