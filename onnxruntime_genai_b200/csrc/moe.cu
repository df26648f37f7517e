// Mixture-of-experts routing around the grouped tcgen05 expert GEMM (ogb_moe_gemm in gemm_tcgen05.cu).
//
//   router logits [T, E] (fp32, from the GEMM)  -- moe_topk -->  expert ids + routing weights [T, k]
//   -- moe_sort -->  token rows grouped by expert: per-expert row ranges, source token of every sorted row,
//                    sorted row of every (token, j) assignment, and the list of token tiles for the GEMM grid
//   -- gather rows, grouped gate/up GEMM (+ clamped SwiGLU), grouped down GEMM --
//   -- moe_combine -->  out[t] = sum_j w[t, j] * y[row(t, j)]  (j order, fp32: deterministic)
//
// Everything stays on the device (no counts are read back), so a decode step with experts replays inside
// a CUDA graph.  With expert parallelism a rank passes its expert range to moe_sort: assignments to other
// ranks' experts get row -1 and are skipped by the combine, whose partial result is then all-reduced.
//
// Reference semantics: the MoE / QMoE contrib op emitted by src/python/py/models/builders/base.py:4176-4408
// (k, normalize_routing_weights, swiglu_fusion) and the router of builders/gptoss.py:653-847.
#include "common.cuh"
#include "kernels.h"

namespace ogb {

// One warp per token.  mode 0: softmax over the k selected logits; mode 1: softmax over all experts, the
// selected probabilities unchanged; mode 2: softmax over all experts, renormalised over the selected.
__global__ void moe_topk_kernel(const float* __restrict__ logits, int ld, int T, int E, int k, int mode, int* __restrict__ topk_idx,
                                float* __restrict__ topk_w) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + size_t(warp) * ld;
  uint32_t taken = 0;  // bit i: this lane's element lane + 32*i is already selected (E <= 1024)
  float all_max = -INFINITY, all_sum = 0.f;
  if (mode != 0) {
    for (int e = lane; e < E; e += 32) all_max = fmaxf(all_max, row[e]);
    all_max = warp_max(all_max);
    for (int e = lane; e < E; e += 32) all_sum += __expf(row[e] - all_max);
    all_sum = warp_sum(all_sum);
  }
  float my_val = 0.f;   // lane j keeps the j-th selected logit
  int my_idx = 0;
  float first = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int i = 0, e = lane; e < E; ++i, e += 32) {
      if (taken >> i & 1) continue;
      const float v = row[e];
      if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);
    if (j == 0) first = best;
    if (lane == j) { my_val = best; my_idx = best_e == 0x7fffffff ? 0 : best_e; }
  }
  float w;
  if (mode == 0) {
    const float ex = lane < k ? __expf(my_val - first) : 0.f;
    w = ex / warp_sum(ex);
  } else {
    const float pr = lane < k ? __expf(my_val - all_max) / all_sum : 0.f;
    w = mode == 2 ? pr / warp_sum(pr) : pr;
  }
  if (lane < k) {
    topk_idx[size_t(warp) * k + lane] = my_idx;
    topk_w[size_t(warp) * k + lane] = w;
  }
}

// Single CTA: counting sort of the n = T*k assignments by expert (local experts [e_lo, e_hi) only).
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ topk_idx, int n, int k, int E, int e_lo, int e_hi, int bt, int* __restrict__ expert_offsets,
                int* __restrict__ sorted_token, int* __restrict__ inv_pos, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                int* __restrict__ tile_rows, int* __restrict__ num_tiles, int max_tiles) {
  extern __shared__ int sm[];
  int* cnt = sm;               // [E]
  int* off = sm + E;           // [E + 1] rows
  int* tbase = off + E + 1;    // [E + 1] tiles
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= e_lo && e < e_hi) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // E is small (<= 1024): a serial scan costs less than a microsecond
    int r = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = r; tbase[e] = t;
      r += cnt[e];
      t += (cnt[e] + bt - 1) / bt;
    }
    off[E] = r; tbase[E] = t;
    *num_tiles = t < max_tiles ? t : max_tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offsets[e] = off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int c = cnt[e];
    for (int j = 0, t = tbase[e]; j * bt < c && t < max_tiles; ++j, ++t) {
      tile_expert[t] = e - e_lo;   // index into this rank's slice of the expert weights
      tile_row0[t] = off[e] + j * bt;
      tile_rows[t] = min(bt, c - j * bt);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;   // reuse as cursors
  __syncthreads();
  // Rows of one expert keep assignment order only up to the atomics' order; every sorted row is computed
  // independently of its neighbours, so the result does not depend on that order.
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = topk_idx[i];
    if (e >= e_lo && e < e_hi) {
      const int pos = off[e] + atomicAdd(&cnt[e], 1);
      sorted_token[pos] = i / k;
      inv_pos[i] = pos;
    } else {
      inv_pos[i] = -1;
    }
  }
  // Rows past the last assignment feed tail tiles of the grouped GEMM: give them a valid source.
  for (int i = off[E] + threadIdx.x; i < n; i += blockDim.x) sorted_token[i] = 0;
}

// out[t, :] = (residual[t, :]) + sum_j w[t, j] * y[inv_pos[t, j], :]   (8 features per thread)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, int ldy, const int* __restrict__ inv_pos,
                                   const float* __restrict__ topk_w, int T, int k, int H, const __nv_bfloat16* __restrict__ residual,
                                   int ldr, __nv_bfloat16* __restrict__ out, int ldo) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 q = *reinterpret_cast<const uint4*>(residual + size_t(t) * ldr + c);
      const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = cc.x; acc[5] = cc.y; acc[6] = d.x; acc[7] = d.y;
    }
    for (int j = 0; j < k; ++j) {
      const int pos = inv_pos[size_t(t) * k + j];
      if (pos < 0) continue;
      const float w = topk_w[size_t(t) * k + j];
      const uint4 q = *reinterpret_cast<const uint4*>(y + size_t(pos) * ldy + c);
      const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
      acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * d.x; acc[7] += w * d.y;
    }
    *reinterpret_cast<uint4*>(out + size_t(t) * ldo + c) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_moe_topk(const float* logits, int ld, int T, int E, int k, int mode, int32_t* topk_idx, float* topk_w, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 1024 || k <= 0 || k > 32 || k > E || mode < 0 || mode > 2) return -1;
  const int threads = 128, warps_per_block = threads / 32;
  moe_topk_kernel<<<(T + warps_per_block - 1) / warps_per_block, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, ld, T, E, k, mode, topk_idx, topk_w);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Upper bound of the tile-list length for n assignments over `experts` experts at token tile `bt`.
OGB_API int ogb_moe_max_tiles(int n, int experts, int bt) {
  const int by_rows = n / bt + experts;   // sum of ceil(c_e / bt) <= n / bt + (experts with a remainder)
  return by_rows < n ? by_rows : n;
}

OGB_API int ogb_moe_sort(const int32_t* topk_idx, int T, int k, int E, int e_lo, int e_hi, int bt, int32_t* expert_offsets,
                         int32_t* sorted_token, int32_t* inv_pos, int32_t* tile_expert, int32_t* tile_row0, int32_t* tile_rows,
                         int32_t* num_tiles, int max_tiles, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 1024 || k <= 0 || bt <= 0 || max_tiles <= 0) return -1;
  const size_t smem = size_t(3 * E + 2) * sizeof(int);
  moe_sort_kernel<<<1, 1024, smem, static_cast<cudaStream_t>(stream)>>>(topk_idx, T * k, k, E, e_lo, e_hi, bt, expert_offsets,
                                                                         sorted_token, inv_pos, tile_expert, tile_row0, tile_rows,
                                                                         num_tiles, max_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_moe_combine(const void* y, int ldy, const int32_t* inv_pos, const float* topk_w, int T, int k, int H,
                            const void* residual, int ldr, void* out, int ldo, void* stream) {
  if (T <= 0) return 0;
  if ((H % 8) || (ldy % 8) || (ldo % 8) || (residual && (ldr % 8))) return -1;
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 15) return -1;
  int threads = (H / 8 + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  moe_combine_kernel<<<T, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), ldy, inv_pos, topk_w, T, k, H, static_cast<const __nv_bfloat16*>(residual), ldr,
      static_cast<__nv_bfloat16*>(out), ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
