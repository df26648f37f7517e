// Gated-delta-rule recurrence of a linear-attention (gated delta net) layer over packed sequences: the LinearAttention contrib op
// with update_rule "gated_delta" that the reference's builder emits for Qwen3-Next / Qwen3.5 style hybrids
// (src/python/py/models/builders/base.py:3419-3452, qwen.py:1842-1860; state handling src/models/recurrent_state.h:12-66).
//
// One CTA = (request, value head, 32 columns of the head's state S [dk, dv]).  The tile lives in registers: a thread keeps 16 to 64
// rows of one column (the rows of a column are split over up to 8 threads); CTAs are small so that several share an SM and their
// load / update / store phases overlap.  The
// per-token update needs no shared-memory traffic for S: with k_t, q_t broadcast from shared memory,
//     S[:, j] *= exp(g);   mem = sum_i S[i, j] k[i];   delta = (v[j] - mem) * beta;   S[i, j] += k[i] * delta;   o[j] = sum_i S[i, j] q[i]
// Tokens of a request are walked in order inside the kernel (a decode step is one token, a prompt chunk many); the state is read
// from / written to the request's slot of the fp32 pool once per launch.  A request whose past length is 0 starts from zero.
#include "common.cuh"
#include "kernels.h"

namespace ogb {

template <int NPT>
__global__ void __launch_bounds__(512) gated_delta_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                         const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                                                         const float* __restrict__ beta, float* __restrict__ state,
                                                         const int32_t* __restrict__ slots, const int32_t* __restrict__ cu_seqlens,
                                                         const int32_t* __restrict__ past_lens, __nv_bfloat16* __restrict__ out,
                                                         int Hk, int Hv, int dv, int dk) {
  // thread (j, sp): column j of the state, rows [sp * NPT, (sp + 1) * NPT); the two dot products of a token (with k, then with q)
  // are summed over the splits through shared memory
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int splits = dk / NPT, CT = blockDim.x / splits;      // CT columns per CTA (blockIdx.z walks the column tiles)
  const int jj = threadIdx.x % CT, j = blockIdx.z * CT + jj, sp = threadIdx.x / CT, n0 = sp * NPT;
  const int hk = h / (Hv / Hk);
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t0 >= t1) return;
  __shared__ float sk[256], sq[256];
  __shared__ float sM[8][128], sO[8][128];
  float* S = state + ((size_t(slots[b]) * Hv + h) * dk + n0) * dv;
  float col[NPT];
  const bool live = j < dv;
  const bool fresh = past_lens[b] == 0;
#pragma unroll
  for (int i = 0; i < NPT; ++i) col[i] = (live && !fresh) ? S[size_t(i) * dv + j] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      sk[i] = bf2f(k[(size_t(t) * Hk + hk) * dk + i]);
      sq[i] = bf2f(q[(size_t(t) * Hk + hk) * dk + i]);
    }
    __syncthreads();
    const float decay = __expf(g[size_t(t) * Hv + h]);
    const float bt = beta[size_t(t) * Hv + h];
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      col[i] *= decay;
      mem = fmaf(col[i], sk[n0 + i], mem);
    }
    if (splits > 1) {
      sM[sp][jj] = mem;
      __syncthreads();
      mem = 0.f;
      for (int s2 = 0; s2 < splits; ++s2) mem += sM[s2][jj];
    }
    const float vj = live ? bf2f(v[(size_t(t) * Hv + h) * dv + j]) : 0.f;
    const float delta = (vj - mem) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      col[i] = fmaf(sk[n0 + i], delta, col[i]);
      o = fmaf(col[i], sq[n0 + i], o);
    }
    if (splits > 1) {
      sO[sp][jj] = o;
      __syncthreads();
      if (sp == 0)
        for (int s2 = 1; s2 < splits; ++s2) o += sO[s2][jj];
    }
    if (live && sp == 0) out[(size_t(t) * Hv + h) * dv + j] = f2bf(o);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[size_t(i) * dv + j] = col[i];
  }
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_gated_delta(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, const int32_t* slots,
                            const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int Hk, int Hv, int dk, int dv, void* stream) {
  if (B <= 0) return 0;
  if (Hk <= 0 || Hv % Hk || dv > 128 || dv <= 0) return -1;
  if (dk < 16 || dk > 256 || (dk & (dk - 1))) return -5;
  // a CTA takes 32 columns of the head's state (all of them when dv is not a multiple of 32): small CTAs, several per SM, so that
  // the load, update and store phases of different CTAs overlap
  const int Pp = (dv % 32 == 0) ? 32 : (dv + 31) / 32 * 32;
  const int ztiles = (dv % 32 == 0) ? dv / 32 : 1;
  int npt = dk < 32 ? dk : 32;
  if (Pp * (dk / npt) > 512) npt = 64;
  const int splits = dk / npt;
  if (splits > 8 || Pp * splits > 512) return -5;
  dim3 grid(B, Hv, ztiles), block(Pp * splits);
  auto s = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k);
  auto V = static_cast<const __nv_bfloat16*>(v);
  auto O = static_cast<__nv_bfloat16*>(out);
  bool ok;
  switch (npt) {
    case 16: ok = launch_pdl(gated_delta_kernel<16>, grid, block, 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv, dk); break;
    case 32: ok = launch_pdl(gated_delta_kernel<32>, grid, block, 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv, dk); break;
    case 64: ok = launch_pdl(gated_delta_kernel<64>, grid, block, 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv, dk); break;
    default: return -5;
  }
  return ok ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------- Mamba-2 selective scan
// The state-space recurrence of a Mamba-2 layer over packed sequences (GraniteMoeHybrid; reference: the Mamba2 branch of
// src/models/recurrent_state.cpp keeps its conv / ssm states, the layer itself is an opaque graph there).  Per head h with
// group gr = h / (heads / groups), per token t, with dt already softplus'ed:
//     S *= exp(dt[t, h] * A[h]);   S[n][p] += dt[t, h] * x[t, h, p] * B[t, gr, n];   y[t, h, p] = sum_n S[n][p] * C[t, gr, n] + D[h] * x[t, h, p]
// state [slots][heads][N][P] fp32, updated in place for the request slots (a request whose past length is 0 starts from a
// zero state).  One CTA per (request, head); a thread keeps 16 to 64 rows of one state column in registers (the rows of a column
// are split over up to 8 threads whose partial sums meet in shared memory), the token's B and C rows sit in
// shared memory; the tokens of a chunk are walked in order.
namespace ogb {
template <int NPT>
__global__ void __launch_bounds__(512) mamba2_scan_kernel(
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ neg_a, const __nv_bfloat16* __restrict__ Bm,
    const __nv_bfloat16* __restrict__ Cm, const float* __restrict__ Dv, float* __restrict__ state, const int32_t* __restrict__ slots,
    const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ past_lens, __nv_bfloat16* __restrict__ out, int heads, int groups, int P,
    int N) {
  // thread (j, sp): column j of the state, rows [sp * NPT, (sp + 1) * NPT); the partial dot products of the splits meet in shared memory
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int splits = N / NPT, Pp = blockDim.x / splits;
  const int j = threadIdx.x % Pp, sp = threadIdx.x / Pp, n0 = sp * NPT;
  const int gr = h / (heads / groups);
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t0 >= t1) return;
  __shared__ float sB[256], sC[256];
  __shared__ float sY[8][128];
  float* S = state + ((size_t(slots[b]) * heads + h) * N + n0) * P;
  float col[NPT];
  const bool live = j < P;
  const bool fresh = past_lens[b] == 0;
#pragma unroll
  for (int i = 0; i < NPT; ++i) col[i] = (live && !fresh) ? S[size_t(i) * P + j] : 0.f;
  const float a = neg_a[h], d = Dv[h];
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      sB[i] = bf2f(Bm[(size_t(t) * groups + gr) * N + i]);
      sC[i] = bf2f(Cm[(size_t(t) * groups + gr) * N + i]);
    }
    __syncthreads();
    const float step = dt[size_t(t) * heads + h];
    const float decay = __expf(step * a);
    const float xj = live ? bf2f(x[(size_t(t) * heads + h) * P + j]) : 0.f;
    const float dx = step * xj;
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      col[i] = fmaf(col[i], decay, dx * sB[n0 + i]);
      y = fmaf(col[i], sC[n0 + i], y);
    }
    if (splits > 1) {
      sY[sp][j] = y;
      __syncthreads();
      if (sp == 0)
        for (int q = 1; q < splits; ++q) y += sY[q][j];
    }
    if (live && sp == 0) out[(size_t(t) * heads + h) * P + j] = f2bf(y + d * xj);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[size_t(i) * P + j] = col[i];
  }
}
}  // namespace ogb

OGB_API int ogb_mamba2_scan(const void* x, const float* dt, const float* neg_a, const void* Bm, const void* Cm, const float* Dv, float* state,
                            const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int heads, int groups,
                            int P, int N, void* stream) {
  if (B <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || P > 128) return -1;
  if (N < 16 || N > 256 || (N & (N - 1))) return -5;
  const int Pp = (P + 31) / 32 * 32;
  int npt = N < 32 ? N : 32;
  if (Pp * (N / npt) > 512) npt = 64;
  const int splits = N / npt;
  if (splits > 8 || Pp * splits > 512) return -5;
  dim3 grid(B, heads), block(Pp * splits);
  auto s = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto Bp = static_cast<const __nv_bfloat16*>(Bm);
  auto Cp = static_cast<const __nv_bfloat16*>(Cm);
  auto O = static_cast<__nv_bfloat16*>(out);
  bool ok;
  switch (npt) {
    case 16: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<16>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N); break;
    case 32: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<32>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N); break;
    case 64: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<64>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N); break;
    default: return -5;
  }
  return ok ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------- state snapshots
// Copies the recurrent states of `count` slots between two pools of the same shape [layers][slots][slot_elems] (or inside
// one): dst[l][dst_slots[i]] = src[l][src_slots[i]].  Speculative decoding saves a request's state before the verification
// pass feeds draft tokens into it and puts it back when some of them are rejected (reference: CopyStateSlotsKernel,
// src/cuda/model_kernels.cu:488-520, used by src/models/recurrent_state.cpp for its snapshot slots).  16 bytes per thread.
namespace ogb {
__global__ void copy_state_slots_kernel(const float4* __restrict__ src, float4* __restrict__ dst, long long layer_vecs, long long slot_vecs,
                                        const int* __restrict__ src_slots, const int* __restrict__ dst_slots, int count) {
  const int pair = blockIdx.y % count, layer = blockIdx.y / count;
  const float4* s = src + size_t(layer) * layer_vecs + size_t(src_slots[pair]) * slot_vecs;
  float4* d = dst + size_t(layer) * layer_vecs + size_t(dst_slots[pair]) * slot_vecs;
  for (long long i = blockIdx.x * blockDim.x + threadIdx.x; i < slot_vecs; i += (long long)gridDim.x * blockDim.x) d[i] = s[i];
}
}  // namespace ogb

OGB_API int ogb_copy_state_slots(const float* src, float* dst, int layers, int slots, long long slot_elems, const int32_t* src_slots,
                                 const int32_t* dst_slots, int count, void* stream) {
  if (count <= 0 || layers <= 0) return 0;
  if (slot_elems <= 0 || (slot_elems % 4) || slots <= 0) return -1;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) return -1;
  if (static_cast<long long>(layers) * count > 65535) return -1;
  const long long slot_vecs = slot_elems / 4;
  const int threads = 256;
  int bx = int((slot_vecs + threads - 1) / threads);
  if (bx > 128) bx = 128;
  ogb::copy_state_slots_kernel<<<dim3(bx, layers * count), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), static_cast<long long>(slots) * slot_vecs, slot_vecs, src_slots, dst_slots, count);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
