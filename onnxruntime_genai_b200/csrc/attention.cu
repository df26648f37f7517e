// Paged variable-length GQA attention (prefill chunks, decode and speculative-verify rows in one
// launch) over a block-table KV cache, with causal masking, sliding window, attention sinks,
// soft-capping and split-KV.
//
// Semantics follow the PagedAttention / GroupQueryAttention contrib ops named by the reference's
// builder (src/python/py/models/builders/base.py:3315-3386, 3484-3536): the packed query holds this
// step's tokens of every request back to back (cumulative_sequence_lengths), the cache already
// holds past_sequence_lengths[b] tokens plus this step's tokens (appended by the RoPE kernel),
// key/value caches are [num_blocks * block_size, kv_heads, head_dim], block_table[b, c] names the
// block that holds positions [c*block_size, (c+1)*block_size); local_window_size > 0 restricts a
// query at position p to keys in (p - window, p], local_window_size < 0 makes every query see all of the request's cached
// keys (bidirectional encoders and cross-attention); `sinks` adds one learned logit per query head
// to the softmax denominator; softcap applies cap * tanh(x / cap) to the scaled scores.
//
// Work decomposition: one CTA = (request, kv head, tile of 64 (or, in decode, 16) query rows, kv split) where a
// "row" is one (query token, query head of the group) pair, so a decode step of a 4:1 GQA model
// keeps its 4 heads in one MMA tile and reads each K/V row once.  K/V tiles of 64 keys are
// gathered through the block table into swizzled shared memory with 16-byte cp.async copies, three tiles in flight per CTA
// (K/V tiles fed by TMA boxes of 16 keys were measured slower for this kernel: 0.52 against 0.68 of the copy bandwidth at 64
// requests x 8 kv heads; the tensor-core prefill kernel in attention_tc.cu is the TMA consumer).
// QK^T and PV run on mma.sync m16n8k16 bf16 with fp32 online softmax.  (The
// tile's M is at most a few rows in decode, far below the 64-row minimum of tcgen05.mma, and
// the kernel is bound by the KV stream, not by tensor throughput.)
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int ATT_BM = 64;   // query rows per CTA (4 warps x 16)
constexpr int ATT_BN = 64;   // keys per tile
constexpr int ATT_THREADS = 128;
constexpr int ATT_STAGES = 3;  // K/V tiles in flight per CTA
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q; int q_stride;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int32_t* cu_seqlens; const int32_t* past_lens;
  const int32_t* block_table; int table_cols; int block_size;
  __nv_bfloat16* out; int out_stride;
  float* part_o; float* part_ml;
  const float* sinks;
  float scale, softcap;
  int window, B, Hq, Hkv, splits, total_rows;
  int* status;       // device status word (bounded waits)
  int chunk;   // > 0: every split owns a fixed range of `chunk` keys (multiple of 64); 0: a request's keys are divided evenly
  // Optional [B] permutation of the requests: blockIdx.z walks `order`, so a caller that lists the requests longest first
  // gets longest-processing-time-first scheduling (CTAs are dispatched in block-index order) - with a mix of 128..2300
  // cached keys per request and fewer than two waves of CTAs the tail of a late long request otherwise sets the time.
  const int32_t* order;
  // 8-bit cache: a (slot, head) row is head_dim int8 values followed by their fp32 scale and 12 bytes of padding
  // (row pitch head_dim + 16); k_cache / v_cache then point at bytes.
  int kv8;
  // > 0: requests with at least this many query rows are left to the tensor-core prefill kernel (attention_tc.cu)
  int skip_rows;
};

template <int SROW>
__device__ __forceinline__ int swz(int row, int chunk) {  // element offset of a 16-byte chunk in a swizzled tile
  return row * SROW + ((((chunk & ~7) | ((chunk ^ row) & 7))) << 3);
}

// DECODE = true: the tile has at most 16 query rows (e.g. one token x a GQA group of up to 16 heads).
// All four warps then share those rows and split the 64 keys of every K/V tile between them
// (16 keys each), keeping private online-softmax state that is merged through shared memory at the
// end.  DECODE = false: each warp owns 16 of the 64 query rows and walks the whole tile.
// KV8 = true: the cache holds int8 rows with an inline scale; raw tiles are staged by cp.async (three in flight) and
// expanded to one bf16 K tile and one bf16 V tile per iteration, so the tensor-core part is the same code.
template <int D, bool DECODE, bool KV8 = false>
__global__ void __launch_bounds__(ATT_THREADS, 2)
paged_attention_kernel(AttnParams p) {
  constexpr int SROW = ((D + 63) / 64) * 64;
  constexpr int CHUNKS = D / 8;     // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;    // k-steps of QK^T
  constexpr int DTILES = D / 8;     // n-tiles of PV
  constexpr int BM = DECODE ? 16 : ATT_BM;
  constexpr int NT = DECODE ? 2 : ATT_BN / 8;  // score n-tiles (8 keys each) per warp and K/V tile
  extern __shared__ __align__(128) uint8_t smem_dyn[];
  uint8_t* smem_raw = smem_dyn;
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  constexpr int BF_STAGES = KV8 ? 1 : ATT_STAGES;
  constexpr int RP = D + 16;                                 // bytes of an int8 cache row (KV8)
  __nv_bfloat16* sK = sQ + BM * SROW;                        // [BF_STAGES][BN][SROW]
  __nv_bfloat16* sV = sK + BF_STAGES * ATT_BN * SROW;        // [BF_STAGES][BN][SROW]
  uint8_t* sRaw = reinterpret_cast<uint8_t*>(sV + BF_STAGES * ATT_BN * SROW);   // KV8: [STAGES][K, V][BN][RP]

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int kvh = blockIdx.y;
  const int bz = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const int b = p.order ? p.order[bz] : bz;
  const int G = p.Hq / p.Hkv;
  const int tok0 = p.cu_seqlens[b];
  const int q_len = p.cu_seqlens[b + 1] - tok0;
  const int rows = q_len * G;
  const int row0 = blockIdx.x * BM;
  if (row0 >= rows) return;
  if (p.skip_rows > 0 && rows >= p.skip_rows) return;
  const int past = p.past_lens[b];
  // window < 0: bidirectional attention over exactly the `past` keys already in the cache (encoder self-attention after
  // its keys were appended, and cross-attention over an encoder's keys); the step's own tokens add no keys.
  const bool full = p.window < 0;
  const int kv_total = full ? past : past + q_len;
  const int32_t* table = p.block_table + size_t(b) * p.table_cols;

  // Key range needed by this tile of rows, then the part of it owned by this split.
  const int last_tq = min(q_len - 1, (row0 + BM - 1) / G);
  int kv_hi = full ? past : past + last_tq + 1;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, past + row0 / G - p.window + 1);
  if (p.splits > 1) {
    // Fixed chunks give every CTA the same amount of work whatever the mix of sequence lengths in the batch (short
    // requests simply use fewer of the launch's splits); the even division suits a batch of similar lengths.
    const int tiles = (kv_total + ATT_BN - 1) / ATT_BN;
    const int per = p.chunk > 0 ? p.chunk : (tiles + p.splits - 1) / p.splits * ATT_BN;
    kv_lo = max(kv_lo, split * per);
    if (split + 1 < p.splits) kv_hi = min(kv_hi, (split + 1) * per);   // the last split takes whatever lies beyond the chunks
  }
  const int tile_begin = kv_lo / ATT_BN;
  const int tile_end = kv_hi > kv_lo ? (kv_hi + ATT_BN - 1) / ATT_BN : tile_begin;
  const int n_tiles = tile_end - tile_begin;
  if (p.splits > 1 && n_tiles == 0) {
    // Nothing in this split's range: mark its partials empty for the combine and leave before any copy is issued.
    for (int r = tid; r < BM; r += ATT_THREADS) {
      const int gr = row0 + r;
      if (gr < rows) {
        float* pm = p.part_ml + (size_t(split) * p.total_rows + size_t(tok0 + gr / G) * p.Hq + kvh * G + gr % G) * 2;
        pm[0] = -INFINITY; pm[1] = 0.f;
      }
    }
    return;
  }

  // element offset of 16-byte chunk `ch` of key row `key` inside a K/V stage
  auto kvoff = [&](int key, int ch) -> int { return swz<SROW>(key, ch); };
  // Each warp copies 16 key rows of the tile.  Lanes 0..15 look up the cache slot of one row each; the
  // copies then walk the warp's rows chunk by chunk with consecutive lanes on consecutive 16-byte
  // chunks, so every warp instruction covers whole 32-byte sectors (full rows for head_dim 128).
  auto load_kv = [&](int tile, int buf) {
    const int jrow = tile * ATT_BN + warp * 16 + (lane & 15);
    int slot = -1;
    if (jrow < kv_hi) slot = table[jrow / p.block_size] * p.block_size + jrow % p.block_size;
    __nv_bfloat16* dk = sK + buf * ATT_BN * SROW;
    __nv_bfloat16* dv = sV + buf * ATT_BN * SROW;
#pragma unroll
    for (int c = 0; c < CHUNKS / 2; ++c) {
      const int item = c * 32 + lane;
      const int kl = item / CHUNKS, ch = item % CHUNKS;
      const int sl = __shfl_sync(0xffffffffu, slot, kl);
      const bool ok = sl >= 0;
      const size_t off = ok ? (size_t(sl) * p.Hkv + kvh) * D + ch * 8 : 0;
      const int key = warp * 16 + kl;
      cp_async16(dk + swz<SROW>(key, ch), p.k_cache + off, ok);
      cp_async16(dv + swz<SROW>(key, ch), p.v_cache + off, ok);
    }
  };

  // KV8: each warp copies the raw bytes of 16 key rows (values + inline scale); rows past the range are zero-filled, which
  // makes their scale 0 and their expanded values 0.
  auto load_kv8 = [&](int tile, int buf) {
    constexpr int RCH = RP / 16;
    const int jrow = tile * ATT_BN + warp * 16 + (lane & 15);
    int slot = -1;
    if (jrow < kv_hi) slot = table[jrow / p.block_size] * p.block_size + jrow % p.block_size;
    const uint8_t* kc = reinterpret_cast<const uint8_t*>(p.k_cache);
    const uint8_t* vc = reinterpret_cast<const uint8_t*>(p.v_cache);
    uint8_t* dk = sRaw + size_t(buf * 2) * ATT_BN * RP;
    uint8_t* dv = dk + ATT_BN * RP;
#pragma unroll
    for (int c = 0; c < (16 * RCH + 31) / 32; ++c) {
      const int item = c * 32 + lane;
      const int kl = min(item / RCH, 15), ch = item % RCH;
      const int sl = __shfl_sync(0xffffffffu, slot, kl);
      if (item < 16 * RCH) {
        const bool ok = sl >= 0;
        const size_t off = ok ? (size_t(sl) * p.Hkv + kvh) * RP + ch * 16 : 0;
        const int key = warp * 16 + kl;
        cp_async16(dk + key * RP + ch * 16, kc + off, ok);
        cp_async16(dv + key * RP + ch * 16, vc + off, ok);
      }
    }
  };
  // KV8: expands raw stage `buf` into the bf16 K and V tiles (value * scale, rounded to bf16).
  auto expand_kv8_rows = [&](int buf, int key0, int nkeys, int worker, int workers) {
    constexpr int VCH = D / 16;          // 16-byte chunks of int8 values per row
    const uint8_t* rk = sRaw + size_t(buf * 2) * ATT_BN * RP;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const uint8_t* src = rk + which * ATT_BN * RP;
      __nv_bfloat16* dst = which ? sV : sK;
      for (int item = worker; item < nkeys * VCH; item += workers) {
        const int key = key0 + item / VCH, c = item % VCH;
        const uint4 raw = *reinterpret_cast<const uint4*>(src + key * RP + c * 16);
        const float sc = *reinterpret_cast<const float*>(src + key * RP + D);
        const int8_t* qv = reinterpret_cast<const int8_t*>(&raw);
        uint4 lo, hi;
        uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
        uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          lw[j] = pack_bf16x2(float(qv[2 * j]) * sc, float(qv[2 * j + 1]) * sc);
          hw[j] = pack_bf16x2(float(qv[8 + 2 * j]) * sc, float(qv[8 + 2 * j + 1]) * sc);
        }
        *reinterpret_cast<uint4*>(dst + swz<SROW>(key, 2 * c)) = lo;
        *reinterpret_cast<uint4*>(dst + swz<SROW>(key, 2 * c + 1)) = hi;
      }
    }
  };

  // Q tile (zero rows beyond the request's rows).
  for (int c = tid; c < BM * CHUNKS; c += ATT_THREADS) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const int gr = row0 + r;
    const bool ok = gr < rows;
    const __nv_bfloat16* src = p.q;
    if (ok) src = p.q + size_t(tok0 + gr / G) * p.q_stride + size_t(kvh * G + gr % G) * D + ch * 8;
    cp_async16(sQ + swz<SROW>(r, ch), src, ok);
  }
  if (KV8) {
    if (n_tiles > 0) load_kv8(tile_begin, 0);
    cp_async_commit();
    if (n_tiles > 1) load_kv8(tile_begin + 1, 1);
    cp_async_commit();
  } else {
    if (n_tiles > 0) load_kv(tile_begin, 0);
    cp_async_commit();
    if (n_tiles > 1) load_kv(tile_begin + 1, 1);
    cp_async_commit();
  }
  const int row_base = DECODE ? 0 : warp * 16;       // first tile row of this warp
  const int key_base = DECODE ? warp * 16 : 0;       // first key (within a K/V tile) of this warp
  const bool warp_active = row0 + row_base < rows;
  // Per-thread rows: r_lo = row_base + g, r_hi = r_lo + 8.
  const int gr_lo = row0 + row_base + g, gr_hi = gr_lo + 8;
  const int qpos_lo = past + gr_lo / G, qpos_hi = past + gr_hi / G;
  const bool valid_lo = gr_lo < rows, valid_hi = gr_hi < rows;

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  uint32_t qf[KSTEPS][4];
  const float sc2 = p.scale * LOG2E;

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it % ATT_STAGES;
    if (KV8) {
      if (it + 2 < n_tiles) load_kv8(tile_begin + it + 2, (it + 2) % ATT_STAGES);
      cp_async_commit();
      cp_async_wait<2>();
      if (DECODE) {
        // decode mode: a warp loads, expands and consumes the same 16 keys of every tile, so after the Q tile (first
        // iteration) the warps need not meet again until the merge
        if (it == 0) __syncthreads(); else __syncwarp();
        expand_kv8_rows(buf, warp * 16, 16, lane, 32);
        __syncwarp();
      } else {
        __syncthreads();        // raw stage `buf` has landed; every warp is done with the bf16 tiles of the last iteration
        expand_kv8_rows(buf, 0, ATT_BN, tid, ATT_THREADS);
        __syncthreads();
      }
    } else {
      if (it + 2 < n_tiles) load_kv(tile_begin + it + 2, (it + 2) % ATT_STAGES);
      cp_async_commit();
      cp_async_wait<2>();
      if (DECODE && it > 0) __syncwarp(); else __syncthreads();   // decode mode: the K/V rows of a warp are its own (see above)
    }
    if (it == 0 && warp_active) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int r = row_base + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(qf[ks], sQ + swz<SROW>(r, ks * 2 + (lane >> 4)));
      }
    }
    if (warp_active) {
      const __nv_bfloat16* tk = sK + (KV8 ? 0 : buf) * ATT_BN * SROW;
      const __nv_bfloat16* tv = sV + (KV8 ? 0 : buf) * ATT_BN * SROW;
      float s[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t kb[4];
          const int key = key_base + (np * 2 + (lane >> 4)) * 8 + (lane & 7);
          ldmatrix_x4(kb, tk + kvoff(key, ks * 2 + ((lane >> 3) & 1)));
          mma_bf16_16816(s[np * 2], qf[ks], kb[0], kb[1]);
          mma_bf16_16816(s[np * 2 + 1], qf[ks], kb[2], kb[3]);
        }
      }
      // scale, softcap, mask, running max
      const int jbase = (tile_begin + it) * ATT_BN + key_base;
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = jbase + nt * 8 + t4 * 2 + (e & 1);
          const bool hi = e >= 2;
          const int qpos = hi ? qpos_hi : qpos_lo;
          bool ok = (hi ? valid_hi : valid_lo) && j >= kv_lo && j < kv_hi && (full || j <= qpos);
          if (p.window > 0) ok = ok && j > qpos - p.window;
          float x = s[nt][e];
          if (p.softcap > 0.f) x = p.softcap * tanhf(x * p.scale / p.softcap) * LOG2E;
          else x *= sc2;
          x = ok ? x : -INFINITY;
          s[nt][e] = x;
          if (hi) mx_hi = fmaxf(mx_hi, x); else mx_lo = fmaxf(mx_lo, x);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float a_lo = exp2f(m_lo - ms_lo), a_hi = exp2f(m_hi - ms_hi);  // m_* = -inf -> 0
      m_lo = mn_lo; m_hi = mn_hi;
      l_lo *= a_lo; l_hi *= a_hi;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= a_lo; o[i][1] *= a_lo; o[i][2] *= a_hi; o[i][3] *= a_hi; }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - ms_lo); s[nt][1] = exp2f(s[nt][1] - ms_lo);
        s[nt][2] = exp2f(s[nt][2] - ms_hi); s[nt][3] = exp2f(s[nt][3] - ms_hi);
        l_lo += s[nt][0] + s[nt][1];
        l_hi += s[nt][2] + s[nt][3];
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          uint32_t vb[4];
          const int key = key_base + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(vb, tv + kvoff(key, dp * 2 + (lane >> 4)));
          mma_bf16_16816(o[dp * 2], pa, vb[0], vb[1]);
          mma_bf16_16816(o[dp * 2 + 1], pa, vb[2], vb[3]);
        }
      }
    }
    if (DECODE) __syncwarp(); else __syncthreads();
  }
  cp_async_wait<0>();

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  if (DECODE) {
    // Merge the four warps' partial states: warp w parks (m, l, O) in shared memory (the K/V stages
    // are idle now), then all threads combine: thread t owns row t/8 and dims [(t%8)*D/8, +D/8).
    __syncthreads();
    float* mo = reinterpret_cast<float*>(sK);          // [4 warps][16 rows][D]
    float* mml = mo + 4 * 16 * D;                      // [4 warps][16 rows][2]
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      *reinterpret_cast<float2*>(mo + (warp * 16 + g) * D + i * 8 + t4 * 2) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * D + i * 8 + t4 * 2) = make_float2(o[i][2], o[i][3]);
    }
    if (t4 == 0) {
      mml[(warp * 16 + g) * 2] = m_lo; mml[(warp * 16 + g) * 2 + 1] = l_lo;
      mml[(warp * 16 + g + 8) * 2] = m_hi; mml[(warp * 16 + g + 8) * 2 + 1] = l_hi;
    }
    __syncthreads();
    const int r = tid >> 3, seg = tid & 7;
    const int gr = row0 + r;
    if (gr >= rows) return;
    constexpr int SEG = D / 8;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    float wgt[4], L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += wgt[w] * mml[(w * 16 + r) * 2 + 1];
    }
    float acc[SEG];
#pragma unroll
    for (int d = 0; d < SEG; ++d) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) a += wgt[w] * mo[(w * 16 + r) * D + seg * SEG + d];
      acc[d] = a;
    }
    const int tq = gr / G, hq = kvh * G + gr % G;
    if (p.splits > 1) {
      const size_t grow = size_t(tok0 + tq) * p.Hq + hq;
      float* po = p.part_o + (size_t(split) * p.total_rows + grow) * D + seg * SEG;
#pragma unroll
      for (int d = 0; d < SEG; ++d) po[d] = acc[d];
      if (seg == 0) {
        float* pm = p.part_ml + (size_t(split) * p.total_rows + grow) * 2;
        pm[0] = M; pm[1] = L;
      }
    } else {
      float scale_o = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[hq] * LOG2E;
        const float mm = fmaxf(M, sk);
        scale_o = exp2f(M - mm);
        L = L * scale_o + exp2f(sk - mm);
      }
      const float inv = L > 0.f ? scale_o / L : 0.f;
      __nv_bfloat16* po = p.out + size_t(tok0 + tq) * p.out_stride + size_t(hq) * D + seg * SEG;
#pragma unroll
      for (int d = 0; d < SEG; d += 2) *reinterpret_cast<uint32_t*>(po + d) = pack_bf16x2(acc[d] * inv, acc[d + 1] * inv);
    }
    return;
  }

  if (!warp_active) return;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int gr = half ? gr_hi : gr_lo;
    if (gr >= rows) continue;
    const int tq = gr / G, hq = kvh * G + gr % G;
    float m = half ? m_hi : m_lo, l = half ? l_hi : l_lo;
    if (p.splits > 1) {
      const size_t grow = size_t(tok0 + tq) * p.Hq + hq;
      float* po = p.part_o + (size_t(split) * p.total_rows + grow) * D;
#pragma unroll
      for (int i = 0; i < DTILES; ++i)
        *reinterpret_cast<float2*>(po + i * 8 + t4 * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      if (t4 == 0) {
        float* pm = p.part_ml + (size_t(split) * p.total_rows + grow) * 2;
        pm[0] = m; pm[1] = l;
      }
    } else {
      float scale_o = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[hq] * LOG2E;
        const float mm = fmaxf(m, sk);
        scale_o = exp2f(m - mm);
        l = l * scale_o + exp2f(sk - mm);
      }
      const float inv = l > 0.f ? scale_o / l : 0.f;
      __nv_bfloat16* po = p.out + size_t(tok0 + tq) * p.out_stride + size_t(hq) * D;
#pragma unroll
      for (int i = 0; i < DTILES; ++i)
        *reinterpret_cast<uint32_t*>(po + i * 8 + t4 * 2) = pack_bf16x2(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
    }
  }
}

// One warp per (token, head) row: merges the split partials (and the sink) into the bf16 output.
template <int D>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, int out_stride,
                                         int total_rows, int Hq, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= total_rows) return;
  const int tok = row / Hq, hq = row % Hq;
  float M = sinks ? sinks[hq] * LOG2E : -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(size_t(s) * total_rows + row) * 2]);
  float L = sinks ? exp2f(sinks[hq] * LOG2E - M) : 0.f;
  constexpr int PER = (D + 31) / 32;
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ml = part_ml + (size_t(s) * total_rows + row) * 2;
    const float m = ml[0];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - M);
    L += w * ml[1];
    const float* po = part_o + (size_t(s) * total_rows + row) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] += w * po[d];
    }
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat16* o = out + size_t(tok) * out_stride + size_t(hq) * D;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    if (d < D) o[d] = f2bf(acc[i] * inv);
  }
}

template <int D, bool DECODE, bool KV8 = false>
static int LaunchAttentionMode(const AttnParams& p, int max_q_len, int cache_slots, cudaStream_t stream) {
  constexpr int SROW = ((D + 63) / 64) * 64;
  constexpr int BM = DECODE ? 16 : ATT_BM;
  constexpr int KV_BYTES = KV8 ? 2 * ATT_BN * SROW * 2 + ATT_STAGES * 2 * ATT_BN * (D + 16) : 2 * ATT_STAGES * ATT_BN * SROW * 2;
  constexpr int SMEM = BM * SROW * 2 + KV_BYTES;
  // decode mode parks the four warps' partial states in the (idle) K/V area, which starts at the K tile and is contiguous
  static_assert(!DECODE || (4 * 16 * D + 4 * 16 * 2) * 4 <= (KV8 ? KV_BYTES : ATT_STAGES * ATT_BN * SROW * 2), "merge buffers must fit in the K/V area");
  auto kern = paged_attention_kernel<D, DECODE, KV8>;
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(kern, SMEM, configured)) return -3;
  const int G = p.Hq / p.Hkv;
  const int q_tiles = (max_q_len * G + BM - 1) / BM;
  dim3 grid(q_tiles, p.Hkv, p.B * p.splits);
  launch_pdl(kern, grid, dim3(ATT_THREADS), SMEM, stream, p);
  if (cudaGetLastError() != cudaSuccess) return -4;
  if (p.splits > 1) {
    const int warps = 4;
    launch_pdl(attention_combine_kernel<D>, dim3((p.total_rows + warps - 1) / warps), dim3(warps * 32), 0, stream,
               static_cast<const float*>(p.part_o), static_cast<const float*>(p.part_ml), p.sinks, p.out, p.out_stride, p.total_rows, p.Hq, p.splits);
    if (cudaGetLastError() != cudaSuccess) return -4;
  }
  return 0;
}

template <int D>
static int LaunchAttention(const AttnParams& p, int max_q_len, int cache_slots, cudaStream_t stream) {
  const int G = p.Hq / p.Hkv;
  if (p.kv8) {
    if (max_q_len * G <= 16) return LaunchAttentionMode<D, true, true>(p, max_q_len, cache_slots, stream);
    return LaunchAttentionMode<D, false, true>(p, max_q_len, cache_slots, stream);
  }
  if (max_q_len * G <= 16) return LaunchAttentionMode<D, true>(p, max_q_len, cache_slots, stream);
  return LaunchAttentionMode<D, false>(p, max_q_len, cache_slots, stream);
}

}  // namespace ogb

using namespace ogb;

// Bytes of fp32 scratch needed for `splits` > 1.
OGB_API long long ogb_attention_scratch_bytes(int total_tokens, int Hq, int D, int splits) {
  if (splits <= 1) return 0;
  return (long long)splits * total_tokens * Hq * (D + 2) * 4;
}

static int PagedAttention(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                          const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                          int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                          int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch,
                          long long scratch_bytes, int cache_slots, const int32_t* order, int* status, void* stream_, int kv_bits,
                          int skip_rows = 0) {
  if (B <= 0 || total_tokens <= 0) return 0;
  if (kv_bits != 16 && kv_bits != 8) return -1;
  if (Hkv <= 0 || Hq % Hkv || (q_stride % 8) || (out_stride % 2)) return -1;
  if (splits < 1) splits = 1;
  if (kv_chunk < 0 || (kv_chunk % ATT_BN)) return -1;
  if (splits > 1 && ogb_attention_scratch_bytes(total_tokens, Hq, D, splits) > scratch_bytes) return -2;
  AttnParams p;
  p.chunk = splits > 1 ? kv_chunk : 0;
  p.status = status;
  p.order = order;
  p.kv8 = kv_bits == 8;
  p.skip_rows = skip_rows;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_stride = q_stride;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache); p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.cu_seqlens = cu_seqlens; p.past_lens = past_lens; p.block_table = block_table; p.table_cols = table_cols;
  p.block_size = block_size; p.out = static_cast<__nv_bfloat16*>(out); p.out_stride = out_stride;
  p.total_rows = total_tokens * Hq;
  p.part_o = static_cast<float*>(scratch);
  p.part_ml = p.part_o ? p.part_o + size_t(splits) * p.total_rows * D : nullptr;
  p.sinks = sinks; p.scale = scale; p.softcap = softcap; p.window = window;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.splits = splits;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  switch (D) {
    case 64: return LaunchAttention<64>(p, max_q_len, cache_slots, stream);
    case 96: return LaunchAttention<96>(p, max_q_len, cache_slots, stream);
    case 128: return LaunchAttention<128>(p, max_q_len, cache_slots, stream);
  }
  return -5;
}

OGB_API int ogb_paged_attention(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                                const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                                int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                                int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch,
                                long long scratch_bytes, int cache_slots, const int32_t* order, int* status, void* stream_) {
  return PagedAttention(q, q_stride, k_cache, v_cache, cu_seqlens, past_lens, block_table, table_cols, block_size, out, out_stride, sinks,
                        scale, softcap, window, B, total_tokens, max_q_len, Hq, Hkv, D, splits, kv_chunk, scratch, scratch_bytes,
                        cache_slots, order, status, stream_, 16);
}

// Same, leaving the requests with at least `skip_rows` query rows to ogb_attention_tc (their output rows are not written here;
// with splits > 1 the combine pass writes unspecified values there, so the tensor-core launch must come afterwards).
OGB_API int ogb_paged_attention_skip(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                                     const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                                     int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                                     int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch,
                                     long long scratch_bytes, int cache_slots, const int32_t* order, int* status, void* stream_, int skip_rows) {
  return PagedAttention(q, q_stride, k_cache, v_cache, cu_seqlens, past_lens, block_table, table_cols, block_size, out, out_stride, sinks,
                        scale, softcap, window, B, total_tokens, max_q_len, Hq, Hkv, D, splits, kv_chunk, scratch, scratch_bytes,
                        cache_slots, order, status, stream_, 16, skip_rows);
}

// Same over an 8-bit cache: rows of head_dim int8 values + fp32 scale + 12 bytes of padding (see AttnParams::kv8).
OGB_API int ogb_paged_attention_kv8(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int32_t* cu_seqlens,
                                    const int32_t* past_lens, const int32_t* block_table, int table_cols, int block_size, void* out,
                                    int out_stride, const float* sinks, float scale, float softcap, int window, int B, int total_tokens,
                                    int max_q_len, int Hq, int Hkv, int D, int splits, int kv_chunk, void* scratch,
                                    long long scratch_bytes, int cache_slots, const int32_t* order, int* status, void* stream_) {
  return PagedAttention(q, q_stride, k_cache, v_cache, cu_seqlens, past_lens, block_table, table_cols, block_size, out, out_stride, sinks,
                        scale, softcap, window, B, total_tokens, max_q_len, Hq, Hkv, D, splits, kv_chunk, scratch, scratch_bytes,
                        cache_slots, order, status, stream_, 8);
}

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (see noalloc.h): the split-KV partials live in a fixed array of
// the library's device image instead of caller-provided scratch.
#include "noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[OGB_NOALLOC_SCRATCH_BYTES];
// Device address of g_noalloc_scratch per device, resolved on the first call with that device current.
static void* g_noalloc_scratch_addr[16] = {};

OGB_API long long ogb_paged_attention_noalloc_required_bytes(int total_tokens, int Hq, int D, int splits) {
  return ogb_attention_scratch_bytes(total_tokens, Hq, D, splits);
}

OGB_API int ogb_paged_attention_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                        const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                                        int table_cols, int block_size, void* out, int out_stride, const float* sinks, float scale,
                                        float softcap, int window, int B, int total_tokens, int max_q_len, int Hq, int Hkv, int D,
                                        int splits, void* stream) {
  if (splits < 1) splits = 1;
  const long long need = ogb_attention_scratch_bytes(total_tokens, Hq, D, splits);
  if (need > OGB_NOALLOC_SCRATCH_BYTES) return OGB_ERR_NOALLOC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return OGB_ERR_NOALLOC_SETUP;
  if (!g_noalloc_scratch_addr[dev]) {
    // In host code `g_noalloc_scratch` names a host-side shadow of the symbol; the kernel needs the
    // address the array has on the current device.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return OGB_ERR_NOALLOC_SETUP;
    g_noalloc_scratch_addr[dev] = p;
  }
  return ogb_paged_attention(q, q_stride, k_cache, v_cache, cu_seqlens, past_lens, block_table, table_cols, block_size, out,
                             out_stride, sinks, scale, softcap, window, B, total_tokens, max_q_len, Hq, Hkv, D, splits, 0,
                             g_noalloc_scratch_addr[dev], OGB_NOALLOC_SCRATCH_BYTES, 0, nullptr, nullptr, stream);
}
