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

struct GdnParams {
  const __nv_bfloat16 *q, *k, *v;     // rows of token t at q + t * tok_stride (+ head offsets): separate tensors or slices of one projection
  long long tok_stride_qk, tok_stride_v;
  const float *g, *beta;              // [T, Hv] log-decay and write strength ...
  const __nv_bfloat16 *b_raw, *a_raw; // ... or (g == null) their raw projections [T, Hv] with a row stride: beta = sigmoid(b),
  long long ba_stride;                //     g = neg_exp_a[h] * softplus(a + dt_bias[h])
  const float *neg_exp_a, *dt_bias;
  int l2norm;                         // q and k are L2-normalised per head here (q then scaled by q_scale)
  float q_scale;
  float* state;
  const int32_t *slots, *cu_seqlens, *past_lens;
  __nv_bfloat16* out;
  int Hk, Hv, dv, dk;
};

template <int NPT>
__global__ void __launch_bounds__(512) gated_delta_kernel(GdnParams p) {
  // thread (j, sp): column j of the state, rows [sp * NPT, (sp + 1) * NPT); the two dot products of a token (with k, then with q)
  // are summed over the splits through shared memory
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int Hk = p.Hk, Hv = p.Hv, dv = p.dv, dk = p.dk;
  const int splits = dk / NPT, CT = blockDim.x / splits;      // CT columns per CTA (blockIdx.z walks the column tiles)
  const int jj = threadIdx.x % CT, j = blockIdx.z * CT + jj, sp = threadIdx.x / CT, n0 = sp * NPT;
  const int hk = h / (Hv / Hk);
  const int t0 = p.cu_seqlens[b], t1 = p.cu_seqlens[b + 1];
  if (t0 >= t1) return;
  __shared__ float sk[256], sq[256];
  __shared__ float sM[8][128], sO[8][128];
  __shared__ float sNorm[2][16];
  float* S = p.state + ((size_t(p.slots[b]) * Hv + h) * dk + n0) * dv;
  float col[NPT];
  const bool live = j < dv;
  const bool fresh = p.past_lens[b] == 0;
#pragma unroll
  for (int i = 0; i < NPT; ++i) col[i] = (live && !fresh) ? S[size_t(i) * dv + j] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    float ssk = 0.f, ssq = 0.f;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      const float kv_ = bf2f(p.k[size_t(t) * p.tok_stride_qk + size_t(hk) * dk + i]);
      const float qv_ = bf2f(p.q[size_t(t) * p.tok_stride_qk + size_t(hk) * dk + i]);
      sk[i] = kv_; sq[i] = qv_;
      ssk += kv_ * kv_; ssq += qv_ * qv_;
    }
    float rk = 1.f, rq = 1.f;
    if (p.l2norm) {
      ssk = warp_sum(ssk); ssq = warp_sum(ssq);
      if ((threadIdx.x & 31) == 0) { sNorm[0][threadIdx.x >> 5] = ssk; sNorm[1][threadIdx.x >> 5] = ssq; }
    }
    __syncthreads();
    if (p.l2norm) {
      float tk = 0.f, tq = 0.f;
      for (int w = 0; w < int(blockDim.x >> 5); ++w) { tk += sNorm[0][w]; tq += sNorm[1][w]; }
      rk = 1.f / fmaxf(sqrtf(tk), 1e-6f);
      rq = p.q_scale / fmaxf(sqrtf(tq), 1e-6f);
    }
    float decay, bt;
    if (p.g) {
      decay = __expf(p.g[size_t(t) * Hv + h]);
      bt = p.beta[size_t(t) * Hv + h];
    } else {
      const float ar = bf2f(p.a_raw[size_t(t) * p.ba_stride + h]) + p.dt_bias[h];
      const float soft = ar > 20.f ? ar : log1pf(__expf(ar));
      decay = __expf(p.neg_exp_a[h] * soft);
      bt = 1.f / (1.f + __expf(-bf2f(p.b_raw[size_t(t) * p.ba_stride + h])));
    }
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
    const float vj = live ? bf2f(p.v[size_t(t) * p.tok_stride_v + size_t(h) * dv + j]) : 0.f;
    const float delta = (vj - mem * rk) * bt * rk;       // the normalised key is rk * sk: once in the read, once in the write
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
    if (live && sp == 0) p.out[(size_t(t) * Hv + h) * dv + j] = f2bf(o * rq);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) S[size_t(i) * dv + j] = col[i];
  }
}

// Output gate of a gated-delta-net layer: per value head, RMS norm of the recurrence output times its weight, times silu of the gate
// projection z (a column slice of the layer's input projection).  One warp per (token, head).
__global__ void gdn_gate_norm_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, long long z_stride,
                                     const float* __restrict__ w, float eps, __nv_bfloat16* __restrict__ out, int rows, int Hv, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = row / Hv, h = row % Hv;
  const __nv_bfloat16* src = o + size_t(row) * dv;
  float x[8];
  float ss = 0.f;
  int n = 0;
  for (int e = lane; e < dv; e += 32, ++n) { x[n] = bf2f(src[e]); ss += x[n] * x[n]; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / dv + eps);
  n = 0;
  for (int e = lane; e < dv; e += 32, ++n) {
    const float zz = bf2f(z[size_t(t) * z_stride + size_t(h) * dv + e]);
    out[size_t(row) * dv + e] = f2bf(x[n] * inv * w[e] * (zz / (1.f + __expf(-zz))));
  }
}

}  // namespace ogb

using namespace ogb;

static int LaunchGatedDelta(GdnParams p, int B, void* stream) {
  if (B <= 0) return 0;
  const int dk = p.dk, dv = p.dv;
  if (p.Hk <= 0 || p.Hv % p.Hk || dv > 128 || dv <= 0) return -1;
  if (dk < 16 || dk > 256 || (dk & (dk - 1))) return -5;
  // a CTA takes 32 columns of the head's state (all of them when dv is not a multiple of 32): small CTAs, several per SM, so that
  // the load, update and store phases of different CTAs overlap
  const int Pp = (dv % 32 == 0) ? 32 : (dv + 31) / 32 * 32;
  const int ztiles = (dv % 32 == 0) ? dv / 32 : 1;
  int npt = dk < 32 ? dk : 32;      // measured at Qwen3.5 shapes: 32 rows per thread 51 us, 16 rows 63 us, 64 rows 54 us (64 requests)
  if (Pp * (dk / npt) > 512) npt = 64;
  const int splits = dk / npt;
  if (splits > 8 || Pp * splits > 512) return -5;
  dim3 grid(B, p.Hv, ztiles), block(Pp * splits);
  auto s = static_cast<cudaStream_t>(stream);
  bool ok;
  switch (npt) {
    case 16: ok = launch_pdl(gated_delta_kernel<16>, grid, block, 0, s, p); break;
    case 32: ok = launch_pdl(gated_delta_kernel<32>, grid, block, 0, s, p); break;
    case 64: ok = launch_pdl(gated_delta_kernel<64>, grid, block, 0, s, p); break;
    default: return -5;
  }
  return ok ? 0 : -4;
}

OGB_API int ogb_gated_delta(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, const int32_t* slots,
                            const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int Hk, int Hv, int dk, int dv, void* stream) {
  GdnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.tok_stride_qk = static_cast<long long>(Hk) * dk; p.tok_stride_v = static_cast<long long>(Hv) * dv;
  p.g = g; p.beta = beta; p.l2norm = 0; p.q_scale = 1.f;
  p.state = state; p.slots = slots; p.cu_seqlens = cu_seqlens; p.past_lens = past_lens; p.out = static_cast<__nv_bfloat16*>(out);
  p.Hk = Hk; p.Hv = Hv; p.dv = dv; p.dk = dk;
  return LaunchGatedDelta(p, B, stream);
}

// The recurrence fed straight from the layer's tensors: q / k / v are column ranges of the convolved projection `conv` [T, row
// stride] (q at q_off, k at k_off, v at v_off), normalised here; the decay and the write strength come from the raw b / a
// projections (column ranges of `ba`, row stride ba_stride) with the layer's -exp(A_log) and dt_bias.
OGB_API int ogb_gated_delta_fused(const void* conv, long long conv_stride, long long q_off, long long k_off, long long v_off, const void* ba,
                                  long long ba_stride, long long b_off, long long a_off, const float* neg_exp_a, const float* dt_bias,
                                  float q_scale, float* state, const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens,
                                  void* out, int B, int Hk, int Hv, int dk, int dv, void* stream) {
  GdnParams p{};
  auto c = static_cast<const __nv_bfloat16*>(conv);
  auto r = static_cast<const __nv_bfloat16*>(ba);
  p.q = c + q_off; p.k = c + k_off; p.v = c + v_off; p.tok_stride_qk = conv_stride; p.tok_stride_v = conv_stride;
  p.g = nullptr; p.beta = nullptr; p.b_raw = r + b_off; p.a_raw = r + a_off; p.ba_stride = ba_stride;
  p.neg_exp_a = neg_exp_a; p.dt_bias = dt_bias; p.l2norm = 1; p.q_scale = q_scale;
  p.state = state; p.slots = slots; p.cu_seqlens = cu_seqlens; p.past_lens = past_lens; p.out = static_cast<__nv_bfloat16*>(out);
  p.Hk = Hk; p.Hv = Hv; p.dv = dv; p.dk = dk;
  return LaunchGatedDelta(p, B, stream);
}

OGB_API int ogb_gdn_gate_norm(const void* o, const void* z, long long z_stride, const float* w, float eps, void* out, int T, int Hv, int dv,
                              void* stream) {
  if (T <= 0) return 0;
  if (dv <= 0 || dv > 256) return -1;
  const int rows = T * Hv;
  return launch_pdl(gdn_gate_norm_kernel, dim3((rows + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(z), z_stride, w, eps,
                    static_cast<__nv_bfloat16*>(out), rows, Hv, dv) ? 0 : -4;
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
    int N, long long x_stride, long long bc_stride, const __nv_bfloat16* __restrict__ dt_raw, long long dt_stride,
    const float* __restrict__ dt_bias) {
  // x_stride / bc_stride: elements between the rows of consecutive tokens in x and in Bm / Cm (tensors of their own, or column
  // ranges of one convolved projection);
  // dt_raw (dt == null): the raw step projection [T, heads] with a row stride, step = softplus(dt_raw + dt_bias[h]) computed here
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
      sB[i] = bf2f(Bm[size_t(t) * bc_stride + size_t(gr) * N + i]);
      sC[i] = bf2f(Cm[size_t(t) * bc_stride + size_t(gr) * N + i]);
    }
    __syncthreads();
    float step;
    if (dt) step = dt[size_t(t) * heads + h];
    else {
      const float r = bf2f(dt_raw[size_t(t) * dt_stride + h]) + dt_bias[h];
      step = r > 20.f ? r : log1pf(__expf(r));
    }
    const float decay = __expf(step * a);
    const float xj = live ? bf2f(x[size_t(t) * x_stride + size_t(h) * P + j]) : 0.f;
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

static int LaunchMamba2(const void* x, const float* dt, const float* neg_a, const void* Bm, const void* Cm, const float* Dv, float* state,
                        const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int heads, int groups, int P,
                        int N, long long x_stride, long long bc_stride, const void* dt_raw, long long dt_stride, const float* dt_bias, void* stream) {
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
  auto R = static_cast<const __nv_bfloat16*>(dt_raw);
  bool ok;
  switch (npt) {
    case 16: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<16>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N, x_stride, bc_stride, R, dt_stride, dt_bias); break;
    case 32: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<32>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N, x_stride, bc_stride, R, dt_stride, dt_bias); break;
    case 64: ok = ogb::launch_pdl(ogb::mamba2_scan_kernel<64>, grid, block, 0, s, X, dt, neg_a, Bp, Cp, Dv, state, slots, cu_seqlens, past_lens, O, heads, groups, P, N, x_stride, bc_stride, R, dt_stride, dt_bias); break;
    default: return -5;
  }
  return ok ? 0 : -4;
}

OGB_API int ogb_mamba2_scan(const void* x, const float* dt, const float* neg_a, const void* Bm, const void* Cm, const float* Dv, float* state,
                            const int32_t* slots, const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int heads, int groups,
                            int P, int N, void* stream) {
  return LaunchMamba2(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu_seqlens, past_lens, out, B, heads, groups, P, N,
                      static_cast<long long>(heads) * P, static_cast<long long>(groups) * N, nullptr, 0, nullptr, stream);
}

// The scan fed straight from the layer's tensors: x / B / C are column ranges of the convolved projection `conv` (row stride
// conv_stride; x at 0, B at heads * P, C after B), the step comes from the raw dt projection (a column range of `proj`) with dt_bias.
OGB_API int ogb_mamba2_scan_fused(const void* conv, long long conv_stride, const void* dt_raw, long long dt_stride, const float* dt_bias,
                                  const float* neg_a, const float* Dv, float* state, const int32_t* slots, const int32_t* cu_seqlens,
                                  const int32_t* past_lens, void* out, int B, int heads, int groups, int P, int N, void* stream) {
  auto c = static_cast<const __nv_bfloat16*>(conv);
  const long long I = static_cast<long long>(heads) * P, GN = static_cast<long long>(groups) * N;
  return LaunchMamba2(c, nullptr, neg_a, c + I, c + I + GN, Dv, state, slots, cu_seqlens, past_lens, out, B, heads, groups, P, N, conv_stride,
                      conv_stride, dt_raw, dt_stride, dt_bias, stream);
}

// Output gate of a Mamba-2 layer: y * silu(z) (z a column range of the input projection), then an RMS norm over the whole width with
// the layer's weight.  One CTA per token.
namespace ogb {
__global__ void __launch_bounds__(256) mamba_gate_norm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                                                             long long z_stride, const float* __restrict__ w, float eps,
                                                             __nv_bfloat16* __restrict__ out, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  __shared__ float part[8];
  float v[16];
  float ss = 0.f;
  int n = 0;
  for (int e = threadIdx.x; e < I; e += blockDim.x, ++n) {
    const float zz = bf2f(z[size_t(t) * z_stride + e]);
    v[n] = bf2f(y[size_t(t) * I + e]) * (zz / (1.f + __expf(-zz)));
    ss += v[n] * v[n];
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < int(blockDim.x >> 5); ++i) tot += part[i];
  const float inv = rsqrtf(tot / I + eps);
  n = 0;
  for (int e = threadIdx.x; e < I; e += blockDim.x, ++n) out[size_t(t) * I + e] = f2bf(v[n] * inv * w[e]);
}
}  // namespace ogb

OGB_API int ogb_mamba_gate_norm(const void* y, const void* z, long long z_stride, const float* w, float eps, void* out, int T, int I, void* stream) {
  if (T <= 0) return 0;
  if (I <= 0 || I > 16 * 256) return -1;
  return ogb::launch_pdl(ogb::mamba_gate_norm_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream),
                         static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z), z_stride, w, eps,
                         static_cast<__nv_bfloat16*>(out), I) ? 0 : -4;
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
