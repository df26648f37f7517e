// Gated-delta-rule recurrence of a linear-attention (gated delta net) layer over packed sequences: the LinearAttention contrib op
// with update_rule "gated_delta" that the reference's builder emits for Qwen3-Next / Qwen3.5 style hybrids
// (src/python/py/models/builders/base.py:3419-3452, qwen.py:1842-1860; state handling src/models/recurrent_state.h:12-66).
//
// One CTA = (request, value head).  Thread j owns column j of the head's state S [dk, dv] in registers (dk <= 128 floats), so the
// per-token update needs no shared-memory traffic for S: with k_t, q_t broadcast from shared memory,
//     S[:, j] *= exp(g);   mem = sum_i S[i, j] k[i];   delta = (v[j] - mem) * beta;   S[i, j] += k[i] * delta;   o[j] = sum_i S[i, j] q[i]
// Tokens of a request are walked in order inside the kernel (a decode step is one token, a prompt chunk many); the state is read
// from / written to the request's slot of the fp32 pool once per launch.  A request whose past length is 0 starts from zero.
#include "common.cuh"
#include "kernels.h"

namespace ogb {

template <int DK>
__global__ void __launch_bounds__(128) gated_delta_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                         const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                                                         const float* __restrict__ beta, float* __restrict__ state,
                                                         const int32_t* __restrict__ slots, const int32_t* __restrict__ cu_seqlens,
                                                         const int32_t* __restrict__ past_lens, __nv_bfloat16* __restrict__ out,
                                                         int Hk, int Hv, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int hk = h / (Hv / Hk);
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t0 >= t1) return;
  __shared__ float sk[DK], sq[DK];
  float* S = state + ((size_t(slots[b]) * Hv + h) * DK) * dv;
  float col[DK];
  const bool live = j < dv;
  const bool fresh = past_lens[b] == 0;
#pragma unroll
  for (int i = 0; i < DK; ++i) col[i] = (live && !fresh) ? S[size_t(i) * dv + j] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      sk[i] = bf2f(k[(size_t(t) * Hk + hk) * DK + i]);
      sq[i] = bf2f(q[(size_t(t) * Hk + hk) * DK + i]);
    }
    __syncthreads();
    const float decay = __expf(g[size_t(t) * Hv + h]);
    const float bt = beta[size_t(t) * Hv + h];
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      col[i] *= decay;
      mem = fmaf(col[i], sk[i], mem);
    }
    const float vj = live ? bf2f(v[(size_t(t) * Hv + h) * dv + j]) : 0.f;
    const float delta = (vj - mem) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      col[i] = fmaf(sk[i], delta, col[i]);
      o = fmaf(col[i], sq[i], o);
    }
    if (live) out[(size_t(t) * Hv + h) * dv + j] = f2bf(o);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[size_t(i) * dv + j] = col[i];
  }
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_gated_delta(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, const int32_t* slots,
                            const int32_t* cu_seqlens, const int32_t* past_lens, void* out, int B, int Hk, int Hv, int dk, int dv, void* stream) {
  if (B <= 0) return 0;
  if (Hk <= 0 || Hv % Hk || dv > 128 || dv <= 0) return -1;
  dim3 grid(B, Hv);
  auto s = static_cast<cudaStream_t>(stream);
  auto Q = static_cast<const __nv_bfloat16*>(q);
  auto K = static_cast<const __nv_bfloat16*>(k);
  auto V = static_cast<const __nv_bfloat16*>(v);
  auto O = static_cast<__nv_bfloat16*>(out);
  bool ok;
  switch (dk) {
    case 16: ok = launch_pdl(gated_delta_kernel<16>, grid, dim3(128), 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv); break;
    case 32: ok = launch_pdl(gated_delta_kernel<32>, grid, dim3(128), 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv); break;
    case 64: ok = launch_pdl(gated_delta_kernel<64>, grid, dim3(128), 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv); break;
    case 128: ok = launch_pdl(gated_delta_kernel<128>, grid, dim3(128), 0, s, Q, K, V, g, beta, state, slots, cu_seqlens, past_lens, O, Hk, Hv, dv); break;
    default: return -5;
  }
  return ok ? 0 : -4;
}
