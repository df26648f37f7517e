// Stand-alone collectives over the symmetric NVLink buffers (the same buffers, flagged lines and call
// counter as the all-reduce fused into the GEMM epilogue, gemm_common.cuh): one-shot all-reduce,
// all-gather and reduce-scatter for tensors that did not come out of a fused GEMM, e.g. the
// expert-parallel combine or the logits gather.  The reference has no communication layer; the bar these
// are measured against is the NCCL call of the same name.
//
// Every thread owns 16-byte vectors of the payload; a vector travels as two flagged lines:
//   all-reduce      push to every rank (plane = source rank) | collect all planes | out = sum (rank order)
//   all-gather      push to every rank (plane = source rank) | collect all planes | out[s * n + i] = plane s
//   reduce-scatter  push vector of slice j to rank j only    | collect all planes | out = sum (rank order)
//   push            push to every rank (plane = source rank) and return: the consumer is the next kernel, a GEMM that
//                   assembles its activation tiles from these lines (all-gather -> GEMM, gemm_tcgen05.cu).  Two pushes
//                   must be separated by a call that waits on every peer (any of the three above, or a fused GEMM).
// Transfers are 16-byte peer stores carrying their own arrival flag; waits are bounded (status word, then the
// kernel finishes without hanging); the last block closes the call's epoch.
//
// NVLS form (when the multicast buffers are registered, see ogb_comm_register_nvls): payload without flags.  Block b of
// every rank owns chunk b of the vectors; the ranks meet at one counter per chunk (multimem.red + bounded acquire wait):
//   all-reduce      copy chunk to the local plane | barrier | sum = multimem.ld_reduce (the switch adds the planes) | out
//                   two-shot for large tensors: each rank sums every world-th vector of the chunk and multimem.st's it to
//                   all ranks | barrier | copy the chunk of sums out
//   all-gather      multimem.st the chunk into plane section `rank` of every rank | barrier | copy the sections out
//   reduce-scatter  copy the chunk of every slice to the local plane | barrier | ld_reduce the chunk of slice `rank`
// The flagged-line form stays for worlds without multicast and for runs in which a rank may leave between steps.
#include <cstdlib>

#include "gemm_common.cuh"
#include "kernels.h"

namespace ogb {

enum CollMode { COLL_ALLREDUCE = 0, COLL_ALLGATHER = 1, COLL_REDUCE_SCATTER = 2, COLL_PUSH = 3 };

constexpr int COLL_THREADS = 256;

// n: bf16 elements per rank plane (all-reduce: tensor size; all-gather: shard size; reduce-scatter: output slice size).
template <int MODE>
__global__ void __launch_bounds__(COLL_THREADS)
collective_kernel(const CommParams c, const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                  const __nv_bfloat16* __restrict__ residual, long long n, int* status) {
  __shared__ uint32_t e_sh;
  if (threadIdx.x == 0) e_sh = comm_open_call(c, gridDim.x);    // the call's epoch; the last block to get here publishes the next
  __syncthreads();
  const uint32_t e = e_sh;
  const uint32_t flag = comm_flag(e);
  const size_t plane_lines = size_t(c.plane_elems) / 4;
  const size_t par_off = size_t(e & 1) * c.world * plane_lines;
  const long long vecs = n / 8;
  const long long stride = (long long)gridDim.x * COLL_THREADS;
  const long long first = (long long)blockIdx.x * COLL_THREADS + threadIdx.x;

  // ---- push
  for (long long v = first; v < vecs; v += stride) {
    const size_t line = par_off + size_t(c.rank) * plane_lines + size_t(v) * 2;
    if (MODE == COLL_REDUCE_SCATTER) {
      for (int r = 0; r < c.world; ++r) {
        const uint4 q = *reinterpret_cast<const uint4*>(in + size_t(r) * n + size_t(v) * 8);
        st_line(c.buf[r] + line, q.x, q.y, flag);
        st_line(c.buf[r] + line + 1, q.z, q.w, flag);
      }
    } else {
      const uint4 q = *reinterpret_cast<const uint4*>(in + size_t(v) * 8);
      for (int r = 0; r < c.world; ++r) {
        st_line(c.buf[r] + line, q.x, q.y, flag);
        st_line(c.buf[r] + line + 1, q.z, q.w, flag);
      }
    }
  }
  // ---- collect the same vectors of every rank from the local receive buffer
  bool dead = false;      // the waits themselves look at the status word from time to time
  const uint4* base = c.buf[c.rank] + par_off;
  for (long long v = first; v < vecs && MODE != COLL_PUSH; v += stride) {
    if (MODE == COLL_ALLGATHER) {
      for (int r = 0; r < c.world; ++r) {
        const uint4 q0 = wait_line(base + size_t(r) * plane_lines + size_t(v) * 2, flag, dead, status);
        const uint4 q1 = wait_line(base + size_t(r) * plane_lines + size_t(v) * 2 + 1, flag, dead, status);
        *reinterpret_cast<uint4*>(out + size_t(r) * n + size_t(v) * 8) = make_uint4(q0.x, q0.z, q1.x, q1.z);
      }
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (residual) {
        const uint4 q = *reinterpret_cast<const uint4*>(residual + size_t(v) * 8);
        const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), cc = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
        acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = cc.x; acc[5] = cc.y; acc[6] = d.x; acc[7] = d.y;
      }
      for (int r = 0; r < c.world; ++r) {   // rank order: bit-identical on every rank
        const uint4 q0 = wait_line(base + size_t(r) * plane_lines + size_t(v) * 2, flag, dead, status);
        const uint4 q1 = wait_line(base + size_t(r) * plane_lines + size_t(v) * 2 + 1, flag, dead, status);
        const float2 a = unpack_bf16x2(q0.x), b = unpack_bf16x2(q0.z), cc = unpack_bf16x2(q1.x), d = unpack_bf16x2(q1.z);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
      }
      *reinterpret_cast<uint4*>(out + size_t(v) * 8) =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// NVLS form of modes 0..2.  n as above; `two_shot` (all-reduce only) selects the owner-reduces-and-multicasts form.
template <int MODE>
__global__ void __launch_bounds__(COLL_THREADS)
nvls_collective_kernel(const CommParams c, const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                       const __nv_bfloat16* __restrict__ residual, long long n, int two_shot, int* status) {
  __shared__ int give_up;
  __shared__ uint32_t e_sh;
  if (threadIdx.x == 0) { give_up = 0; e_sh = comm_open_call(c, gridDim.x); }
  __syncthreads();
  const uint32_t e = e_sh;
  const size_t par = size_t(e & 1) * size_t(c.nv_plane_elems);
  const long long vecs = n / 8;
  const long long per = (vecs + gridDim.x - 1) / gridDim.x;
  const long long v0 = (long long)blockIdx.x * per, v1 = min(vecs, v0 + per);
  auto rank_barrier = [&](int phase) {
    __syncthreads();     // every thread's stores of this phase are ordered before thread 0's release
    if (threadIdx.x == 0 && !give_up && !nvls_arrive_and_wait(c, phase, blockIdx.x, status)) give_up = 1;
    __syncthreads();
    return give_up == 0;
  };
  auto add8 = [&](uint4 q, long long v) {   // + residual, in fp32
    if (!residual) return q;
    const uint4 r = *reinterpret_cast<const uint4*>(residual + size_t(v) * 8);
    auto add2 = [](uint32_t a, uint32_t b) { const float2 x = unpack_bf16x2(a), y = unpack_bf16x2(b); return pack_bf16x2(x.x + y.x, x.y + y.y); };
    return make_uint4(add2(q.x, r.x), add2(q.y, r.y), add2(q.z, r.z), add2(q.w, r.w));
  };
  if (MODE == COLL_ALLREDUCE) {
    for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
      *reinterpret_cast<uint4*>(c.nv_data + par + size_t(v) * 8) = *reinterpret_cast<const uint4*>(in + size_t(v) * 8);
    if (rank_barrier(0)) {
      if (!two_shot) {
        for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
          *reinterpret_cast<uint4*>(out + size_t(v) * 8) = add8(multimem_ld_reduce_bf16x8(c.nv_data_mc + par + size_t(v) * 8), v);
      } else {
        for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
          if (int((v / COLL_THREADS + v) % c.world) == c.rank)
            multimem_st_b128(c.nv_out_mc + par + size_t(v) * 8, multimem_ld_reduce_bf16x8(c.nv_data_mc + par + size_t(v) * 8));
        if (rank_barrier(1))
          for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
            *reinterpret_cast<uint4*>(out + size_t(v) * 8) = add8(ld_line(reinterpret_cast<const uint4*>(c.nv_out + par + size_t(v) * 8)), v);
      }
    }
  } else if (MODE == COLL_ALLGATHER) {
    for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
      multimem_st_b128(c.nv_out_mc + par + size_t(c.rank) * n + size_t(v) * 8, *reinterpret_cast<const uint4*>(in + size_t(v) * 8));
    if (rank_barrier(0))
      for (int r = 0; r < c.world; ++r)
        for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
          *reinterpret_cast<uint4*>(out + size_t(r) * n + size_t(v) * 8) =
              ld_line(reinterpret_cast<const uint4*>(c.nv_out + par + size_t(r) * n + size_t(v) * 8));
  } else {   // reduce-scatter
    for (int r = 0; r < c.world; ++r)
      for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
        *reinterpret_cast<uint4*>(c.nv_data + par + size_t(r) * n + size_t(v) * 8) = *reinterpret_cast<const uint4*>(in + size_t(r) * n + size_t(v) * 8);
    if (rank_barrier(0))
      for (long long v = v0 + threadIdx.x; v < v1; v += COLL_THREADS)
        *reinterpret_cast<uint4*>(out + size_t(v) * 8) = add8(multimem_ld_reduce_bf16x8(c.nv_data_mc + par + size_t(c.rank) * n + size_t(v) * 8), v);
  }
}

}  // namespace ogb

using namespace ogb;

// mode 0 all-reduce (in/out n elements), 1 all-gather (in n, out world * n), 2 reduce-scatter (in world * n, out n),
// 3 push (in n; no output: the next kernel reads the lines).
// n must be a multiple of 8 and at most the registered plane size; pointers 16-byte aligned.  residual (modes 0, 2) is
// added to the sum.  Uses the symmetric buffers registered for `device` with ogb_comm_register.
OGB_API int ogb_collective(int mode, const void* in, void* out, const void* residual, long long n, int device, int* status,
                           int sm_count, void* stream_) {
  const CommParams* cp = ogb_comm_params(device);
  if (!cp || cp->world < 1 || !cp->buf[0]) return -2;
  if (n <= 0) return 0;
  if (n % 8) return -1;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 15) return -1;
  if (mode != COLL_PUSH && !out) return -1;
  const int nvls_env = int(ogb_comm_options()[0]);
  const long long two_shot_bytes = ogb_comm_options()[1];
  const long long nv_need = mode == COLL_ALLREDUCE ? n : n * cp->world;
  if (nvls_env && cp->nv_data_mc && mode != COLL_PUSH && nv_need <= cp->nv_plane_elems) {
    long long nb = (n / 8 + COLL_THREADS * 4 - 1) / (COLL_THREADS * 4);   // ~4 vectors per thread
    const long long ncap = sm_count * 2 < NV_MAX_CTAS ? sm_count * 2 : NV_MAX_CTAS;
    if (nb > ncap) nb = ncap;
    if (nb < 1) nb = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    const __nv_bfloat16* i = static_cast<const __nv_bfloat16*>(in);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const __nv_bfloat16* r = static_cast<const __nv_bfloat16*>(residual);
    const int two_shot = (cp->world > 2 && (long long)cp->world * n * 2 > two_shot_bytes) ? 1 : 0;
    switch (mode) {
      case COLL_ALLREDUCE: nvls_collective_kernel<COLL_ALLREDUCE><<<unsigned(nb), COLL_THREADS, 0, st>>>(*cp, i, o, r, n, two_shot, status); break;
      case COLL_ALLGATHER: nvls_collective_kernel<COLL_ALLGATHER><<<unsigned(nb), COLL_THREADS, 0, st>>>(*cp, i, o, nullptr, n, 0, status); break;
      case COLL_REDUCE_SCATTER: nvls_collective_kernel<COLL_REDUCE_SCATTER><<<unsigned(nb), COLL_THREADS, 0, st>>>(*cp, i, o, r, n, 0, status); break;
      default: return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (n > cp->plane_elems) return -1;
  long long blocks = (n / 8 + COLL_THREADS * 2 - 1) / (COLL_THREADS * 2);   // ~2 vectors per thread
  const long long cap = sm_count * 2;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const __nv_bfloat16* i = static_cast<const __nv_bfloat16*>(in);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* r = static_cast<const __nv_bfloat16*>(residual);
  switch (mode) {
    case COLL_ALLREDUCE: collective_kernel<COLL_ALLREDUCE><<<unsigned(blocks), COLL_THREADS, 0, stream>>>(*cp, i, o, r, n, status); break;
    case COLL_ALLGATHER: collective_kernel<COLL_ALLGATHER><<<unsigned(blocks), COLL_THREADS, 0, stream>>>(*cp, i, o, nullptr, n, status); break;
    case COLL_REDUCE_SCATTER: collective_kernel<COLL_REDUCE_SCATTER><<<unsigned(blocks), COLL_THREADS, 0, stream>>>(*cp, i, o, r, n, status); break;
    case COLL_PUSH: collective_kernel<COLL_PUSH><<<unsigned(blocks), COLL_THREADS, 0, stream>>>(*cp, i, nullptr, nullptr, n, status); break;
    default: return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
