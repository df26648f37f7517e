// Bandwidth-bound per-token kernels: embedding gather, RMSNorm / LayerNorm with fused residual add,
// RoPE + (optional per-head q/k RMSNorm) + paged KV-cache append, SiLU*mul, logits edits.
//
// Reference semantics: SkipSimplifiedLayerNormalization returns both the normalised tensor and the
// residual sum (src/python/py/models/builders/base.py:2342-2403); RotaryEmbedding uses
// cos/sin caches of shape [ctx, rot/2] with an interleaved flag (base.py:2565-2637); PagedAttention
// appends the new K/V rows at slots derived from the block table (base.py:3484-3536).
#include <cuda_fp16.h>
#include "common.cuh"
#include "kernels.h"

namespace ogb {

// ------------------------------------------------------------------------------------ embedding
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const uint4* __restrict__ table, uint4* __restrict__ out,
                                 int vec_per_row, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = table + size_t(id) * vec_per_row;
  uint4* dst = out + size_t(t) * vec_per_row;
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
    uint4 v = __ldg(src + i);
    if (scale != 1.f) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = unpack_bf16x2(w[k]);
        w[k] = pack_bf16x2(f.x * scale, f.y * scale);
      }
    }
    dst[i] = v;
  }
}

// Embedding rows gathered straight from an int4 block-32 weight (GatherBlockQuantized over the tied LM-head weight):
// q [vocab, K / 2] bytes (low nibble = even k), scales fp16 [vocab, K / 32], zero points packed two per byte
// [vocab, ceil(K / 64)] or null (8).  out[t, k] = (q - zp) * scale * mult, restated in bf16 exactly like the int4 GEMM's
// dequantisation.  One CTA per token, eight values (four bytes) per thread.
__global__ void embedding_q4_kernel(const int32_t* __restrict__ ids, const uint32_t* __restrict__ q, const __half* __restrict__ scales,
                                    const uint8_t* __restrict__ zps, uint4* __restrict__ out, int K, int vocab, float mult) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const int nb = K / 32, zp_pitch = (nb + 1) / 2;
  const uint32_t* row = q + size_t(id) * (K / 8);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint32_t w = __ldg(row + i);
    const int blk = i / 4;
    const float sc = __half2float(scales[size_t(id) * nb + blk]);     // the checkpoint's fp16 scale, exactly
    int zp = 8;
    if (zps) { const uint8_t z = zps[size_t(id) * zp_pitch + blk / 2]; zp = (blk & 1) ? (z >> 4) : (z & 0xF); }
    uint4 o;
    __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int nib = (w >> (4 * j)) & 0xF;
      oe[j] = f2bf(float(nib - zp) * sc * mult);
    }
    out[size_t(t) * (K / 8) + i] = o;
  }
}

// ------------------------------------------------------------------------------------ norm
// One CTA per row. h = x (+ residual_in); residual_out = h (optional); out = norm(h) * w (+ b).
// The row is kept in registers (up to 2 vectors of 8 bf16 per thread, hidden size <= 16384).
// comb.y != nullptr: x is not read; the row is the weighted sum of the experts' output rows (the combine step of a
// mixture-of-experts layer: row t = sum_j topk_w[t, j] * y[inv_pos[t, j]], rows of experts that are not local skipped),
// summed in fp32 in j order and rounded to bf16 exactly as the stand-alone combine kernel stores it.
struct NormCombine {
  const __nv_bfloat16* y;
  const int* inv_pos;
  const float* topk_w;
  int ldy, k;
};
template <bool LAYERNORM>
__global__ void __launch_bounds__(1024) norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res_in,
                                                    uint4* __restrict__ res_out, const uint4* __restrict__ weight,
                                                    const uint4* __restrict__ bias, uint4* __restrict__ out, int H, float eps,
                                                    const NormCombine comb) {
  constexpr int MAXV = 2;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, nvec = H / 8;
  const uint4* xr = x + size_t(row) * nvec;
  float v[MAXV][8];
  float sum = 0.f, sumsq = 0.f;
  int cnt = 0;
  for (int i = threadIdx.x; i < nvec && cnt < MAXV; i += blockDim.x, ++cnt) {
    uint4 a;
    if (comb.y) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < comb.k; ++j) {
        const int pos = comb.inv_pos[size_t(row) * comb.k + j];
        if (pos < 0) continue;
        const float w = comb.topk_w[size_t(row) * comb.k + j];
        const uint4 q = *reinterpret_cast<const uint4*>(comb.y + size_t(pos) * comb.ldy + i * 8);
        const float2 q0 = unpack_bf16x2(q.x), q1 = unpack_bf16x2(q.y), q2 = unpack_bf16x2(q.z), q3 = unpack_bf16x2(q.w);
        acc[0] += w * q0.x; acc[1] += w * q0.y; acc[2] += w * q1.x; acc[3] += w * q1.y;
        acc[4] += w * q2.x; acc[5] += w * q2.y; acc[6] += w * q3.x; acc[7] += w * q3.y;
      }
      a = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    } else {
      a = xr[i];
    }
    const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a);
    uint4 r = make_uint4(0, 0, 0, 0);
    if (res_in) r = res_in[size_t(row) * nvec + i];
    const uint32_t* rw = reinterpret_cast<const uint32_t*>(&r);
    uint4 hs;
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hs);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 fa = unpack_bf16x2(aw[k]), fr = unpack_bf16x2(rw[k]);
      float h0 = fa.x + fr.x, h1 = fa.y + fr.y;
      hw[k] = pack_bf16x2(h0, h1);
      if (res_in) {  // the residual stream is stored in bf16: normalise what is stored
        float2 q = unpack_bf16x2(hw[k]);
        h0 = q.x; h1 = q.y;
      }
      v[cnt][2 * k] = h0; v[cnt][2 * k + 1] = h1;
      sum += h0 + h1;
      sumsq += h0 * h0 + h1 * h1;
    }
    if (res_out) res_out[size_t(row) * nvec + i] = hs;
  }
  __shared__ float red[2][32];
  sum = warp_sum(sum);
  sumsq = warp_sum(sumsq);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) { red[0][warp] = sum; red[1][warp] = sumsq; }
  __syncthreads();
  if (warp == 0) {
    float a = lane < nw ? red[0][lane] : 0.f, b = lane < nw ? red[1][lane] : 0.f;
    a = warp_sum(a); b = warp_sum(b);
    if (lane == 0) { red[0][0] = a; red[1][0] = b; }
  }
  __syncthreads();
  const float mean = LAYERNORM ? red[0][0] / H : 0.f;
  const float var = LAYERNORM ? fmaxf(red[1][0] / H - mean * mean, 0.f) : red[1][0] / H;
  const float inv = rsqrtf(var + eps);
  cnt = 0;
  for (int i = threadIdx.x; i < nvec && cnt < MAXV; i += blockDim.x, ++cnt) {
    uint4 w = weight[i];
    const uint32_t* ww = reinterpret_cast<const uint32_t*>(&w);
    uint4 b = make_uint4(0, 0, 0, 0);
    if (bias) b = bias[i];
    const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 fw = unpack_bf16x2(ww[k]), fb = unpack_bf16x2(bw[k]);
      ow[k] = pack_bf16x2((v[cnt][2 * k] - mean) * inv * fw.x + fb.x, (v[cnt][2 * k + 1] - mean) * inv * fw.y + fb.y);
    }
    out[size_t(row) * nvec + i] = o;
  }
}

// ------------------------------------------------------------------------------------ RoPE + KV append
// One warp per (token, head) of the packed [T, (Hq + 2*Hkv) * D] activation.  Q heads are rotated in
// place; K heads are rotated and written to the cache slot; V heads are copied to the cache slot.
struct RopeParams {
  __nv_bfloat16* qkv;
  int qkv_stride;            // elements between tokens
  const int32_t* positions;  // [T]
  const int32_t* slots;      // [T] cache slot (block * block_size + offset); < 0 skips the append
  const float* cos_cache;    // [ctx, rot/2]
  const float* sin_cache;
  __nv_bfloat16* k_cache;    // [slots, Hkv, D]
  __nv_bfloat16* v_cache;
  const __nv_bfloat16* q_norm_w;  // optional [D]
  const __nv_bfloat16* k_norm_w;  // optional [D]
  float norm_eps;
  int T, Hq, Hkv, D, rot, interleaved, max_pos;
  int kv8;   // 8-bit cache: rows of D int8 values + fp32 scale (absmax / 127 of the row) + 12 bytes of padding
  // Multimodal RoPE (Qwen2-VL): three position components per token ([3, T]: temporal, height, width); rotary pair i takes
  // component 0 below sec0, component 1 below sec1, component 2 above.  Null: the single `positions` array.
  // Interleaved layout (Qwen3-VL), passed as sec0 < 0: pair i takes the height component when i % 3 == 1 and i < -sec0, the width
  // component when i % 3 == 2 and i < sec1, the temporal component otherwise (-sec0 = 3 * height pairs, sec1 = 3 * width pairs).
  const int32_t* positions3;
  int sec0, sec1;
};

__device__ __forceinline__ int rope_component(const RopeParams& p, int i) {
  if (p.sec0 >= 0) return i < p.sec0 ? 0 : (i < p.sec1 ? 1 : 2);
  const int m = i % 3;
  return (m == 1 && i < -p.sec0) ? 1 : ((m == 2 && i < p.sec1) ? 2 : 0);
}

__device__ __forceinline__ int rope_pos(const RopeParams& p, int t, int i) {
  int pos = p.positions3 ? p.positions3[size_t(rope_component(p, i)) * p.T + t] : p.positions[t];
  return pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
}

__global__ void __launch_bounds__(256) rope_kv_kernel(RopeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float buf[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hkv;
  const long item = long(blockIdx.x) * 8 + warp;
  if (item >= long(p.T) * heads) return;
  const int t = int(item / heads), h = int(item % heads);
  __nv_bfloat16* src = p.qkv + size_t(t) * p.qkv_stride + size_t(h) * p.D;
  float* v = buf[warp];
  const bool is_q = h < p.Hq, is_k = !is_q && h < p.Hq + p.Hkv;
  float ss = 0.f;
  for (int e = lane; e < p.D; e += 32) { float x = bf2f(src[e]); v[e] = x; ss += x * x; }
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / p.D + p.norm_eps);
    __syncwarp();
    for (int e = lane; e < p.D; e += 32) v[e] = bf2f(f2bf(v[e] * inv * bf2f(nw[e])));
  }
  __syncwarp();
  const int slot = p.slots ? p.slots[t] : -1;
  __nv_bfloat16* dst;
  if (is_q) dst = src;
  else {
    if (slot < 0) return;
    const int kvh = is_k ? h - p.Hq : h - p.Hq - p.Hkv;
    if (p.kv8) {
      // rotate in the row buffer, then quantise the whole row against its largest magnitude
      if (is_k && p.rot > 0) {
        const int half = p.rot / 2;
        for (int i = lane; i < half; i += 32) {
          const int a = p.interleaved ? 2 * i : i, b = p.interleaved ? 2 * i + 1 : i + half;
          const size_t ci = size_t(rope_pos(p, t, i)) * half + i;
          const float x1 = v[a], x2 = v[b], c = p.cos_cache[ci], s = p.sin_cache[ci];
          v[a] = x1 * c - x2 * s;
          v[b] = x2 * c + x1 * s;
        }
        __syncwarp();
      }
      float amax = 0.f;
      for (int e = lane; e < p.D; e += 32) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      // correctly rounded divisions (the library is built with fast-math): the stored scale is the same on every path
      const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
      const float inv = __fdiv_rn(1.f, scale);
      int8_t* row = reinterpret_cast<int8_t*>(is_k ? p.k_cache : p.v_cache) + (size_t(slot) * p.Hkv + kvh) * (p.D + 16);
      for (int e = lane; e < p.D; e += 32) row[e] = int8_t(max(-127, min(127, __float2int_rn(v[e] * inv))));
      if (lane == 0) *reinterpret_cast<float*>(row + p.D) = scale;
      return;
    }
    dst = (is_k ? p.k_cache : p.v_cache) + (size_t(slot) * p.Hkv + kvh) * p.D;
  }
  if ((is_q || is_k) && p.rot > 0) {
    const int half = p.rot / 2;
    for (int i = lane; i < half; i += 32) {
      const int a = p.interleaved ? 2 * i : i, b = p.interleaved ? 2 * i + 1 : i + half;
      const size_t ci = size_t(rope_pos(p, t, i)) * half + i;
      const float x1 = v[a], x2 = v[b], c = p.cos_cache[ci], s = p.sin_cache[ci];
      dst[a] = f2bf(x1 * c - x2 * s);
      dst[b] = f2bf(x2 * c + x1 * s);
    }
    for (int e = p.rot + lane; e < p.D; e += 32) dst[e] = f2bf(v[e]);
  } else if (!is_q || nw) {
    for (int e = lane; e < p.D; e += 32) dst[e] = f2bf(v[e]);
  }
}

// ------------------------------------------------------------------------------------ SiLU * mul
// out[t, i] = act(x[t, i]) * x[t, I + i];  act 0 = SiLU, 1 = GELU(tanh)
__global__ void act_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int T, int I, int act) {
  const long n = long(T) * I;
  for (long idx = long(blockIdx.x) * blockDim.x + threadIdx.x; idx < n; idx += long(gridDim.x) * blockDim.x) {
    const long t = idx / I, i = idx % I;
    const float g = bf2f(x[t * 2 * I + i]), u = bf2f(x[t * 2 * I + I + i]);
    float a;
    if (act == 0) a = g / (1.f + __expf(-g));
    else a = 0.5f * g * (1.f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
    out[idx] = f2bf(a * u);
  }
}

// ------------------------------------------------------------------------------------ plain activation
// out[i] = act(x[i]) for the fc1 -> act -> fc2 MLPs (phi, gpt2): 0 SiLU, 1 GELU(tanh), 2 ReLU, 3 GELU(erf).
// Eight bf16 per thread (16-byte loads and stores); n is a multiple of 8.
__global__ void act_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, long n_vec, int act) {
  pdl_launch_dependents(); pdl_wait();
  for (long idx = long(blockIdx.x) * blockDim.x + threadIdx.x; idx < n_vec; idx += long(gridDim.x) * blockDim.x) {
    uint4 v = x[idx];
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = bf2f(e[j]);
      float a;
      if (act == 0) a = g / (1.f + __expf(-g));
      else if (act == 1) a = 0.5f * g * (1.f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
      else if (act == 2) a = fmaxf(g, 0.f);
      else if (act == 4) { const float r = fmaxf(g, 0.f); a = r * r; }
      else a = 0.5f * g * (1.f + erff(g * 0.70710678f));
      e[j] = f2bf(a);
    }
    out[idx] = v;
  }
}

// ------------------------------------------------------------------------------------ gated short convolution
// Hybrid (LFM2) layers: y[t] = c[t] * sum_{k < L} w[:, L-1-k] * (b*x)[pos(t) - k] (+ bias), channels independent.
// The product b*x of every position lives in a paged cache addressed like the key/value cache ([slots, C]); a token
// writes its own entry and reads the entries of the L-1 positions before it: from the packed input when that position
// belongs to this step (another CTA may not have written it yet), otherwise from the cache through the block table.
// One CTA per token, eight channels per thread.
struct ShortConvParams {
  const uint4* bcx; int bcx_stride;       // [T, 3C] bf16, stride in elements
  const __nv_bfloat16* weight;            // [C, L]
  const __nv_bfloat16* bias;              // [C] or null
  uint4* cache;                           // [slots, C]
  const int32_t* slots; const int32_t* positions; const int32_t* cu_seqlens; const int32_t* past_lens;
  const int32_t* block_table; int table_cols, block_size;
  uint4* out;                             // [T, C]
  int T, B, C, L;
  int plain;                              // no gates: bcx holds x alone ([T, C], the causal convolutions of the recurrent layer kinds)
  int silu;                               // SiLU on the output
};

__global__ void __launch_bounds__(256) short_conv_kernel(ShortConvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  // the request this token belongs to: last r with cu_seqlens[r] <= t
  int lo = 0, hi = p.B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (p.cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int r = lo, pos = p.positions[t], past = p.past_lens[r], t0 = p.cu_seqlens[r];
  const int slot = p.slots[t];
  const int nvec = p.C / 8;
  const int32_t* table = p.block_table + size_t(r) * p.table_cols;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = p.bias ? bf2f(p.bias[v * 8 + j]) : 0.f;
    uint4 mine = make_uint4(0, 0, 0, 0);
    for (int k = 0; k < p.L; ++k) {
      const int q = pos - k;
      if (q < 0) break;
      uint4 e;
      if (q >= past) {
        // produced in this step by token t0 + (q - past): recompute b * x from the packed input
        const uint4* row = p.bcx + size_t(t0 + (q - past)) * (p.bcx_stride / 8);
        if (p.plain) {
          e = row[v];
        } else {
          const uint4 bb = row[v], xx = row[2 * nvec + v];
          const __nv_bfloat16* be = reinterpret_cast<const __nv_bfloat16*>(&bb);
          const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&xx);
          __nv_bfloat16* ee = reinterpret_cast<__nv_bfloat16*>(&e);
#pragma unroll
          for (int j = 0; j < 8; ++j) ee[j] = f2bf(bf2f(be[j]) * bf2f(xe[j]));
        }
        if (k == 0) mine = e;
      } else {
        const int blk = table[q / p.block_size];
        e = p.cache[(size_t(blk) * p.block_size + q % p.block_size) * nvec + v];
      }
      const __nv_bfloat16* ee = reinterpret_cast<const __nv_bfloat16*>(&e);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += bf2f(p.weight[size_t(v * 8 + j) * p.L + (p.L - 1 - k)]) * bf2f(ee[j]);
    }
    if (slot >= 0) p.cache[size_t(slot) * nvec + v] = mine;
    uint4 o;
    __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&o);
    if (!p.plain) {
      const uint4 cc = (p.bcx + size_t(t) * (p.bcx_stride / 8))[nvec + v];
      const __nv_bfloat16* ce = reinterpret_cast<const __nv_bfloat16*>(&cc);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= bf2f(ce[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = f2bf(p.silu ? acc[j] / (1.f + __expf(-acc[j])) : acc[j]);
    p.out[size_t(t) * nvec + v] = o;
  }
}

// ------------------------------------------------------------------------------------ decode look-ahead
// Turns the packed inputs of a decode step (one token per request) into those of the next one on the device: the token
// just sampled becomes the input, position, past length and sampling counter move on by one, and the cache slot of the
// new position is looked up in the request's block table (which already lists the block of that position).  The engine
// uses it to enqueue step n + 1 before the ids of step n have reached the host.
__global__ void decode_advance_kernel(const int32_t* __restrict__ sampled, int32_t* input_ids, int32_t* positions, int32_t* past_lens,
                                      int32_t* slot_mapping, int32_t* sample_pos, const int32_t* __restrict__ block_table,
                                      int table_cols, int block_size, int B) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int pos = positions[i] + 1;
  input_ids[i] = sampled[i];
  positions[i] = pos;
  past_lens[i] += 1;
  sample_pos[i] += 1;
  const int col = pos / block_size;
  const int blk = col < table_cols ? block_table[size_t(i) * table_cols + col] : -1;
  slot_mapping[i] = blk < 0 ? -1 : blk * block_size + pos % block_size;
}

// ------------------------------------------------------------------------------------ logits edits
// A sparse list of (row, token) edits: op 0 sets the logit to -FLT_MAX (min_length / no-repeat-ngram /
// banned tokens), op 1 applies the repetition penalty (x < 0 ? x * v : x / v).  O(list) instead of
// the O(vocab * length) scan the reference does on the GPU (src/cuda/search_cuda.cu:160-189).
__global__ void logits_edit_kernel(float* logits, int vocab, const int32_t* rows, const int32_t* tokens, const int32_t* ops,
                                   const float* values, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok = tokens[i];
  if (tok < 0 || tok >= vocab) return;
  float* p = logits + size_t(rows[i]) * vocab + tok;
  if (ops[i] == 0) *p = -3.402823466e+38f;
  else { const float x = *p, v = values[i]; *p = x < 0.f ? x * v : x / v; }
}

// logits[row, v] = -FLT_MAX where bit v of the row's mask is clear (grammar constraints).
// mask_rows maps a logits row to a mask row (-1 = unconstrained).
__global__ void logits_bitmask_kernel(float* logits, int vocab, const uint32_t* mask, const int32_t* mask_rows, int words) {
  const int row = blockIdx.y;
  const int mr = mask_rows ? mask_rows[row] : row;
  if (mr < 0) return;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vocab) return;
  if (!((mask[size_t(mr) * words + (v >> 5)] >> (v & 31)) & 1u)) logits[size_t(row) * vocab + v] = -3.402823466e+38f;
}

// Cast rows of bf16 to fp32 (logits hand-off when a model computes bf16 logits).
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long n) {
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) out[i] = bf2f(in[i]);
}

// Gather rows: out[i, :] = in[rows[i], :] (16-byte vectors).
__global__ void gather_rows_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ rows, uint4* __restrict__ out, int vec_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows[blockIdx.x];
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) out[size_t(blockIdx.x) * vec_per_row + i] = in[size_t(r) * vec_per_row + i];
}

// Gather rows with a bf16 -> fp16 conversion (activations of the fp16 form of the packed FP4 expert GEMM).
__global__ void gather_rows_f16_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ rows, uint4* __restrict__ out, int vec_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows[blockIdx.x];
  for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
    uint4 v = in[size_t(r) * vec_per_row + i];
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const __half2 h = __floats2half2_rn(f.x, f.y);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    out[size_t(blockIdx.x) * vec_per_row + i] = v;
  }
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_embedding(const int32_t* ids, const void* table, void* out, int T, int H, int vocab, float scale, void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -1;
  launch_pdl(embedding_kernel, dim3(T), dim3(min(256, H / 8)), 0, static_cast<cudaStream_t>(stream),
      ids, static_cast<const uint4*>(table), static_cast<uint4*>(out), H / 8, vocab, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_embedding_q4(const int32_t* ids, const void* q, const void* scales, const void* zps, void* out, int T, int K, int vocab,
                             float mult, void* stream) {
  if (T <= 0) return 0;
  if (K % 32) return -1;
  return launch_pdl(embedding_q4_kernel, dim3(T), dim3(min(256, K / 8)), 0, static_cast<cudaStream_t>(stream), ids,
                    static_cast<const uint32_t*>(q), static_cast<const __half*>(scales), static_cast<const uint8_t*>(zps),
                    static_cast<uint4*>(out), K, vocab, mult) ? 0 : -4;
}

static int LaunchNorm(const void* x, const void* residual_in, void* residual_out, const void* weight, const void* bias, void* out, int rows,
                      int H, float eps, int layernorm, const NormCombine& comb, void* stream) {
  if (rows <= 0) return 0;
  if (H % 8 || H / 8 > 8 * 1024) return -1;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  if (nvec > threads * 2) return -1;
  auto s = static_cast<cudaStream_t>(stream);
  if (layernorm)
    launch_pdl(norm_kernel<true>, dim3(rows), dim3(threads), 0, s, static_cast<const uint4*>(x), static_cast<const uint4*>(residual_in),
               static_cast<uint4*>(residual_out), static_cast<const uint4*>(weight), static_cast<const uint4*>(bias), static_cast<uint4*>(out),
               H, eps, comb);
  else
    launch_pdl(norm_kernel<false>, dim3(rows), dim3(threads), 0, s, static_cast<const uint4*>(x), static_cast<const uint4*>(residual_in),
               static_cast<uint4*>(residual_out), static_cast<const uint4*>(weight), static_cast<const uint4*>(bias), static_cast<uint4*>(out),
               H, eps, comb);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_norm(const void* x, const void* residual_in, void* residual_out, const void* weight, const void* bias,
                     void* out, int rows, int H, float eps, int layernorm, void* stream) {
  return LaunchNorm(x, residual_in, residual_out, weight, bias, out, rows, H, eps, layernorm, NormCombine{nullptr, nullptr, nullptr, 0, 0}, stream);
}

// ogb_norm over rows that are still spread over the experts' outputs: row t = sum_j topk_w[t, j] * y[inv_pos[t, j]]
// (what ogb_moe_combine would have written), then the residual add and the norm in the same launch.
OGB_API int ogb_norm_moe_combine(const void* y, int ldy, const int32_t* inv_pos, const float* topk_w, int k, const void* residual_in,
                                 void* residual_out, const void* weight, const void* bias, void* out, int rows, int H, float eps,
                                 int layernorm, void* stream) {
  if ((ldy % 8) || k <= 0 || (reinterpret_cast<uintptr_t>(y) & 15)) return -1;
  return LaunchNorm(nullptr, residual_in, residual_out, weight, bias, out, rows, H, eps, layernorm,
                    NormCombine{static_cast<const __nv_bfloat16*>(y), inv_pos, topk_w, ldy, k}, stream);
}

OGB_API int ogb_rope_kv_append(void* qkv, int qkv_stride, const int32_t* positions, const int32_t* slots, const float* cos_cache,
                               const float* sin_cache, void* k_cache, void* v_cache, const void* q_norm_w, const void* k_norm_w,
                               float norm_eps, int T, int Hq, int Hkv, int D, int rot, int interleaved, int max_pos, void* stream) {
  return ogb_rope_kv_append_bits(qkv, qkv_stride, positions, slots, cos_cache, sin_cache, k_cache, v_cache, q_norm_w, k_norm_w, norm_eps, T,
                                 Hq, Hkv, D, rot, interleaved, max_pos, 16, nullptr, 0, 0, stream);
}

// kv_bits 16: bf16 cache rows; 8: int8 rows with an inline scale (row pitch D + 16 bytes, D a multiple of 16).
OGB_API int ogb_rope_kv_append_bits(void* qkv, int qkv_stride, const int32_t* positions, const int32_t* slots, const float* cos_cache,
                                    const float* sin_cache, void* k_cache, void* v_cache, const void* q_norm_w, const void* k_norm_w,
                                    float norm_eps, int T, int Hq, int Hkv, int D, int rot, int interleaved, int max_pos, int kv_bits,
                                    const int32_t* positions3, int sec0, int sec1, void* stream) {
  if (T <= 0) return 0;
  if (D > 256 || rot > D || (rot & 1)) return -1;
  if (kv_bits != 16 && (kv_bits != 8 || (D % 16))) return -1;
  RopeParams p;
  p.kv8 = kv_bits == 8;
  p.positions3 = positions3; p.sec0 = sec0; p.sec1 = sec1;
  p.qkv = static_cast<__nv_bfloat16*>(qkv); p.qkv_stride = qkv_stride; p.positions = positions; p.slots = slots;
  p.cos_cache = cos_cache; p.sin_cache = sin_cache;
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache); p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_w); p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_w);
  p.norm_eps = norm_eps; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rot = rot; p.interleaved = interleaved; p.max_pos = max_pos;
  const long items = long(T) * (Hq + 2 * Hkv);
  launch_pdl(rope_kv_kernel, dim3(unsigned((items + 7) / 8)), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_act_mul(const void* x, void* out, int T, int I, int act, void* stream) {
  if (T <= 0) return 0;
  const long n = long(T) * I;
  long nb = (n + 255) / 256; int blocks = int(nb < 148 * 16 ? nb : 148 * 16);
  act_mul_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                         static_cast<__nv_bfloat16*>(out), T, I, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_act(const void* x, void* out, long long n, int act, void* stream) {
  if (n <= 0) return 0;
  if (n % 8) return -2;
  const long nv = n / 8;
  long nb = (nv + 255) / 256; int blocks = int(nb < 148 * 8 ? nb : 148 * 8);
  return launch_pdl(act_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint4*>(x), static_cast<uint4*>(out), nv, act) ? 0 : -4;
}

static int LaunchShortConv(const void* bcx, int bcx_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                           const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                           int table_cols, int block_size, void* out, int T, int B, int C, int L, int plain, int silu, void* stream);

OGB_API int ogb_short_conv(const void* bcx, int bcx_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                           const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                           int table_cols, int block_size, void* out, int T, int B, int C, int L, void* stream) {
  return LaunchShortConv(bcx, bcx_stride, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, table_cols, block_size, out,
                         T, B, C, L, 0, 0, stream);
}

// The causal depthwise convolution without gates (x [T, C] with a row stride, e.g. a slice of a wider projection), optional SiLU:
// the CausalConvWithState op of the gated-delta-net and Mamba-2 layers over the same paged window.
OGB_API int ogb_causal_conv(const void* x, int x_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                            const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                            int table_cols, int block_size, void* out, int T, int B, int C, int L, int silu, void* stream) {
  if (reinterpret_cast<uintptr_t>(x) & 15) return -1;
  return LaunchShortConv(x, x_stride, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, table_cols, block_size, out,
                         T, B, C, L, 1, silu, stream);
}

static int LaunchShortConv(const void* bcx, int bcx_stride, const void* weight, const void* bias, void* cache, const int32_t* slots,
                           const int32_t* positions, const int32_t* cu_seqlens, const int32_t* past_lens, const int32_t* block_table,
                           int table_cols, int block_size, void* out, int T, int B, int C, int L, int plain, int silu, void* stream) {
  if (T <= 0) return 0;
  if (B <= 0 || (C % 8) || (bcx_stride % 8) || L < 1 || L > 16 || block_size <= 0) return -1;
  ShortConvParams p;
  p.bcx = static_cast<const uint4*>(bcx); p.bcx_stride = bcx_stride;
  p.weight = static_cast<const __nv_bfloat16*>(weight); p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.cache = static_cast<uint4*>(cache); p.slots = slots; p.positions = positions; p.cu_seqlens = cu_seqlens; p.past_lens = past_lens;
  p.block_table = block_table; p.table_cols = table_cols; p.block_size = block_size; p.out = static_cast<uint4*>(out);
  p.T = T; p.B = B; p.C = C; p.L = L; p.plain = plain; p.silu = silu;
  const int threads = min(256, max(32, (C / 8 + 31) / 32 * 32));
  return launch_pdl(short_conv_kernel, dim3(T), dim3(threads), 0, static_cast<cudaStream_t>(stream), p) ? 0 : -4;
}

OGB_API int ogb_decode_advance(const int32_t* sampled, int32_t* input_ids, int32_t* positions, int32_t* past_lens, int32_t* slot_mapping,
                               int32_t* sample_pos, const int32_t* block_table, int table_cols, int block_size, int B, void* stream) {
  if (B <= 0) return 0;
  if (block_size <= 0 || table_cols <= 0) return -1;
  return launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), sampled, input_ids,
                    positions, past_lens, slot_mapping, sample_pos, block_table, table_cols, block_size, B) ? 0 : -4;
}

OGB_API int ogb_logits_edit(float* logits, int vocab, const int32_t* rows, const int32_t* tokens, const int32_t* ops,
                            const float* values, int n, void* stream) {
  if (n <= 0) return 0;
  logits_edit_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, vocab, rows, tokens, ops, values, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_logits_bitmask(float* logits, int rows, int vocab, const uint32_t* mask, const int32_t* mask_rows, void* stream) {
  if (rows <= 0) return 0;
  const int words = (vocab - 1) / 32 + 1;
  dim3 grid((vocab + 255) / 256, rows);
  logits_bitmask_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, vocab, mask, mask_rows, words);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_bf16_to_f32(const void* in, float* out, long long n, void* stream) {
  if (n <= 0) return 0;
  long long nb = (n + 255) / 256; int blocks = int(nb < 148 * 16 ? nb : 148 * 16);
  bf16_to_f32_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(in), out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_gather_rows_f16(const void* in, const int32_t* rows, void* out, int n_rows, int row_bytes, void* stream) {
  if (n_rows <= 0) return 0;
  if (row_bytes % 16) return -1;
  launch_pdl(gather_rows_f16_kernel, dim3(n_rows), dim3(min(256, row_bytes / 16)), 0, static_cast<cudaStream_t>(stream),
      static_cast<const uint4*>(in), rows, static_cast<uint4*>(out), row_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_gather_rows(const void* in, const int32_t* rows, void* out, int n_rows, int row_bytes, void* stream) {
  if (n_rows <= 0) return 0;
  if (row_bytes % 16) return -1;
  launch_pdl(gather_rows_kernel, dim3(n_rows), dim3(min(256, row_bytes / 16)), 0, static_cast<cudaStream_t>(stream),
      static_cast<const uint4*>(in), rows, static_cast<uint4*>(out), row_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
