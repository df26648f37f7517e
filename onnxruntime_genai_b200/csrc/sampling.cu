// Token selection on the device: one kernel per step for a whole batch with PER-ROW parameters
// (top_k, top_p, temperature, seed, position), plus top-k scoring for beam search and the
// speculative-verification kernel.
//
// Semantics follow the reference pipeline (src/sampling_distribution.h:233-297 on the host,
// src/cuda/cuda_sampling.cu:90-239 on the device): restrict to the k largest logits, softmax with
// temperature, keep the shortest prefix (by descending probability) whose mass reaches top_p,
// renormalise, draw.  Differences by design:
//   * no sort: the kept set is described by a key threshold found with an 8-bit radix select (by
//     count for top-k, by probability mass for top-p); the draw is a prefix scan over the kept
//     set in index order;
//   * probability masses are accumulated in 40-bit fixed point with integer atomics, so the
//     result is bit-reproducible from run to run and independent of how rows are batched;
//   * randomness is Philox4x32-10 keyed by (seed, sequence position): stateless, so rolling a
//     step back needs no RNG bookkeeping, and a request samples the same tokens alone or batched;
//   * rows are not bucketed by (k, p, T) (reference: src/cuda/interface.cpp:156-359): every row
//     reads its own parameters.
#include "common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int SAMP_THREADS = 1024;
constexpr float SAMP_LOG2E = 1.4426950408889634f;
constexpr float MASS_SCALE = 1099511627776.0f;  // 2^40
constexpr int SMALL_K = 1024;  // top-k sets up to this size are finished on a sorted list in shared memory

__device__ __forceinline__ uint32_t to_key(float f) {  // order-preserving float -> uint
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowCtx {
  const float* x;
  int n;
  float mx;      // row maximum
  float inv_t2;  // log2(e) / temperature
  // top-k membership: key > tk, or key == tk and index <= tk_idx
  uint32_t tk;
  int tk_idx;
  bool use_k;
  __device__ __forceinline__ bool in_k(int i, uint32_t key) const {
    return !use_k || key > tk || (key == tk && i <= tk_idx);
  }
  __device__ __forceinline__ unsigned long long mass(float v) const {
    return (unsigned long long)(exp2f((v - mx) * inv_t2) * MASS_SCALE);
  }
};

struct SelectShared {
  unsigned long long hist[256];   // combined histogram of the current pass
  unsigned long long want, above, ties;
  uint32_t prefix, mask;
  unsigned long long warp_tot[32];
  unsigned long long carry;
  int result;
};

// Radix select over the row, 8 bits per pass.  MASS = false: weights are 1 (count); MASS = true:
// fixed-point probability mass.  Each warp owns a private 256-bin histogram (`priv`, dynamic shared
// memory, [warps][256]); lanes that fall into the same bin are combined with match.any first, so
// the hot bins (most float keys share their top byte) cost one plain add per warp, no atomics.
// On return sh.prefix is the threshold key T, sh.above the weight of members with key > T,
// sh.want the weight still needed from members with key == T and sh.ties their total weight.
template <bool MASS>
__device__ void radix_select(const RowCtx& c, SelectShared& sh, unsigned long long* priv, unsigned long long want) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  unsigned long long* mine = priv + warp * 256;
  if (tid == 0) { sh.want = want; sh.above = 0; sh.prefix = 0; sh.mask = 0; sh.ties = 0; }
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = tid; b < nwarps * 256; b += blockDim.x) priv[b] = 0;
    __syncthreads();
    const uint32_t prefix = sh.prefix, mask = sh.mask;
    // The row is read in batches of UNR independent loads per thread: one trip to L2 per batch, not per element.
    constexpr int UNR = 8;
    for (int base = 0; base < c.n; base += UNR * blockDim.x) {
      float vals[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int i = base + u * blockDim.x + tid;
        vals[u] = i < c.n ? c.x[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int i = base + u * blockDim.x + tid;
        uint32_t bin = 0xFFFFFFFFu;
        unsigned long long w = 0;
        if (i < c.n) {
          const float v = vals[u];
          const uint32_t key = to_key(v);
          if ((key & mask) == prefix && c.in_k(i, key)) {
            w = MASS ? c.mass(v) : 1ull;
            if (w) bin = (key >> shift) & 255;
          }
        }
        if (!__any_sync(0xffffffffu, bin != 0xFFFFFFFFu)) continue;  // later passes: most warps see no candidate
        const unsigned grp = __match_any_sync(0xffffffffu, bin);
        if (bin != 0xFFFFFFFFu) {
          unsigned long long sum;
          if (MASS) {
            const unsigned lo = __reduce_add_sync(grp, unsigned(w & 0xFFFFFu));
            const unsigned hi = __reduce_add_sync(grp, unsigned(w >> 20));
            sum = ((unsigned long long)hi << 20) + lo;
          } else {
            sum = __popc(grp);
          }
          if (lane == __ffs(grp) - 1) mine[bin] += sum;
        }
        __syncwarp();
      }
    }
    __syncthreads();
    for (int b = tid; b < 256; b += blockDim.x) {
      unsigned long long t = 0;
      for (int w = 0; w < nwarps; ++w) t += priv[w * 256 + b];
      sh.hist[b] = t;
    }
    __syncthreads();
    if (tid < 32) {
      // lane l owns bins [8l, 8l+8); suffix sums from the top bin downwards
      unsigned long long local = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) local += sh.hist[tid * 8 + j];
      unsigned long long suffix = local;  // inclusive suffix over lanes >= tid
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned long long up = __shfl_down_sync(0xffffffffu, suffix, o);
        if (tid + o < 32) suffix += up;
      }
      const unsigned long long w = sh.want;
      const unsigned long long higher = suffix - local;  // weight in lanes above this one
      const bool here = higher < w && suffix >= w;
      const unsigned found_mask = __ballot_sync(0xffffffffu, here);
      if (found_mask == 0) {
        // fewer members than requested: take everything (threshold = lowest non-empty bin)
        const unsigned nonempty = __ballot_sync(0xffffffffu, local > 0);
        if (nonempty && tid == __ffs(nonempty) - 1) {
          int bin = 0;
          for (int j = 0; j < 8; ++j) if (sh.hist[tid * 8 + j]) { bin = tid * 8 + j; break; }
          unsigned long long cum = higher;
          for (int j = 7; j >= 0; --j) if (tid * 8 + j > bin) cum += sh.hist[tid * 8 + j];
          sh.above += cum;
          sh.want = sh.hist[bin];
          sh.ties = sh.hist[bin];
          sh.prefix |= uint32_t(bin) << shift;
          sh.mask |= 255u << shift;
        }
      } else if (here) {
        unsigned long long cum = higher;
        int bin = tid * 8;
        for (int j = 7; j >= 0; --j) {
          const unsigned long long h = sh.hist[tid * 8 + j];
          if (cum + h >= w) { bin = tid * 8 + j; break; }
          cum += h;
        }
        sh.above += cum;
        sh.want = w - cum;
        sh.ties = sh.hist[bin];
        sh.prefix |= uint32_t(bin) << shift;
        sh.mask |= 255u << shift;
      }
    }
    __syncthreads();
  }
}

// Block-wide inclusive scan of one value per thread (index order = thread order).
__device__ __forceinline__ unsigned long long block_scan_incl(unsigned long long v, SelectShared& sh, unsigned long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned long long up = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += up;
  }
  if (lane == 31) sh.warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < (blockDim.x >> 5) ? sh.warp_tot[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned long long up = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += up;
    }
    sh.warp_tot[lane] = t;  // inclusive totals of warps
  }
  __syncthreads();
  const unsigned long long before = warp ? sh.warp_tot[warp - 1] : 0;
  total = sh.warp_tot[(blockDim.x >> 5) - 1];
  return v + before;
}

// Smallest index I such that members with key == T and index <= I carry at least `want` weight
// (weight 1 per member when !MASS).  Used only when ties straddle a threshold.
template <bool MASS>
__device__ int tie_index_cut(const RowCtx& c, SelectShared& sh, uint32_t T, unsigned long long want, bool k_member_only) {
  if (threadIdx.x == 0) { sh.carry = 0; sh.result = c.n - 1; }
  __syncthreads();
  for (int base = 0; base < c.n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    unsigned long long w = 0;
    if (i < c.n) {
      const float v = c.x[i];
      const uint32_t key = to_key(v);
      if (key == T && (!k_member_only || c.in_k(i, key))) w = MASS ? c.mass(v) : 1ull;
    }
    unsigned long long total;
    const unsigned long long incl = block_scan_incl(w, sh, total);
    const unsigned long long carry = sh.carry;
    const bool hit = w && carry + incl >= want && carry + incl - w < want;
    if (hit) sh.result = i;
    __syncthreads();
    const bool done = carry + total >= want;
    if (threadIdx.x == 0) sh.carry = carry + total;
    __syncthreads();
    if (done) break;
  }
  return sh.result;
}

struct SampleParams {
  const float* logits;
  long long row_stride;
  int vocab, rows;
  const int32_t* top_k; const float* top_p; const float* temperature;
  const unsigned long long* seeds; const int32_t* positions;
  int32_t* out;
};


// The k <= SMALL_K candidates of a row as a sorted list in shared memory (descending value, ties by lower
// index) with their fixed-point masses: thread j < m owns entry j (mass w, inclusive prefix incl); `kept` is
// the mass of the prefix that survives top-p (entries with incl <= kept are the sampled distribution).
struct SmallList {
  float* sv; int* si;
  int m;
  unsigned long long w, incl, kept;
};

// Cluster helpers (a row may be shared by the CTAs of a thread-block cluster: see sample_kernel).
__device__ __forceinline__ unsigned samp_cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned samp_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void samp_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t samp_dsmem(const void* local, unsigned rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}

// C > 1: the row's first two passes are divided between the C CTAs of the cluster (contiguous slices); every CTA appends its
// candidates to the list of CTA 0 through distributed shared memory, and CTA 0 alone finishes the row (the others return
// from the caller after the cluster barrier at the end of the collection).
__device__ void small_list(const RowCtx& c, SelectShared& sh, unsigned long long* priv, int* cand_n, int k, float top_p, SmallList& L,
                           unsigned C, unsigned crank, float* slice_bound) {
  const int tid = threadIdx.x, n = c.n;
  const float* x = c.x;
  float* cv = reinterpret_cast<float*>(priv);            // candidate values   [SMALL_K]
  int* ci = reinterpret_cast<int*>(cv + SMALL_K);        // candidate indices  [SMALL_K]
  float* sv = reinterpret_cast<float*>(ci + SMALL_K);    // sorted values
  int* si = reinterpret_cast<int*>(sv + SMALL_K);        // sorted indices
  const int per = C > 1 ? ((n + int(C) - 1) / int(C) + 3) & ~3 : n;
  const int lo = min(n, int(crank) * per), hi = min(n, lo + per);

  // ---- fast path: two light passes.  The k-th largest of the per-thread maxima (distinct elements of the row) is a
  // lower bound of the k-th largest element, so everything >= it is a superset of the top-k set; for k << n and
  // interleaved indexing that superset is a small multiple of k.  If it does not fit the list the exact radix
  // select below takes over, so the result never depends on which path ran.  (Cluster: each CTA has such a bound from
  // its own slice; the largest of them is used by all.)
  float tmax = -INFINITY;
  for (int base = lo; base < hi; base += 8 * blockDim.x) {
    float vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x + tid;
      vals[u] = i < hi ? x[i] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) tmax = fmaxf(tmax, vals[u]);
  }
  sv[tid] = tmax;   // blockDim.x == SMALL_K
  if (tid == 0) { *cand_n = 0; sh.result = 0; }
  // bitonic sort of the 1024 maxima, descending: 55 compare-exchange steps, one element per thread
  for (int size = 2; size <= SAMP_THREADS; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      const int partner = tid ^ stride;
      if (partner > tid) {
        const bool desc = (tid & size) == 0;
        const float a = sv[tid], b = sv[partner];
        if ((a < b) == desc && a != b) { sv[tid] = b; sv[partner] = a; }
      }
    }
  }
  __syncthreads();
  float t0 = sv[k - 1];
  if (C > 1) {
    if (tid == 0) *slice_bound = t0;
    samp_cluster_sync();          // every CTA's bound is published; CTA 0's candidate counter is zero
    for (unsigned r = 0; r < C; ++r) {
      float o;
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(o) : "r"(samp_dsmem(slice_bound, r)) : "memory");
      t0 = fmaxf(t0, o);
    }
  }
  __syncthreads();
  const uint32_t r_n = samp_dsmem(cand_n, 0), r_cv = samp_dsmem(cv, 0), r_ci = samp_dsmem(ci, 0);
  for (int base = lo; base < hi; base += 8 * blockDim.x) {
    float vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x + tid;
      vals[u] = i < hi ? x[i] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x + tid;
      if (i < hi && vals[u] >= t0) {
        if (C > 1) {
          int slot;
          asm volatile("atom.shared::cluster.add.u32 %0, [%1], 1;" : "=r"(slot) : "r"(r_n) : "memory");
          if (slot < SMALL_K) {
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r_cv + uint32_t(slot) * 4), "f"(vals[u]) : "memory");
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(r_ci + uint32_t(slot) * 4), "r"(i) : "memory");
          }
        } else {
          const int slot = atomicAdd(cand_n, 1);
          if (slot < SMALL_K) { cv[slot] = vals[u]; ci[slot] = i; }
        }
      }
    }
  }
  if (C > 1) {
    samp_cluster_sync();          // all candidates are in CTA 0's list
    if (crank != 0) return;
  }
  __syncthreads();
  int m = *cand_n;
  __syncthreads();
  if (m > SMALL_K || m < k) {
    // ---- exact path: radix select of the k-th key, then collect exactly the k members
    radix_select<false>(c, sh, priv, (unsigned long long)k);
    const uint32_t T = sh.prefix;
    const unsigned long long need = sh.want, ties = sh.ties;
    __syncthreads();
    int cut = n;
    if (need < ties) cut = tie_index_cut<false>(c, sh, T, need, false);  // ties straddle the threshold: keep the lowest indices
    __syncthreads();
    if (tid == 0) *cand_n = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 8 * blockDim.x) {
      float vals[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * blockDim.x + tid;
        vals[u] = i < n ? x[i] : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * blockDim.x + tid;
        const uint32_t key = to_key(vals[u]);
        if (i < n && (key > T || (key == T && i <= cut))) {
          const int slot = atomicAdd(cand_n, 1);
          if (slot < SMALL_K) { cv[slot] = vals[u]; ci[slot] = i; }
        }
      }
    }
    __syncthreads();
    m = min(*cand_n, SMALL_K);
  }
  // rank sort: descending value, ascending index (deterministic whatever order the slots were filled in); the first k
  // ranks are the top-k set (ties at the boundary go to the lowest indices)
  if (tid < m) {
    const float v = cv[tid];
    const int idx = ci[tid];
    int rank = 0;
    for (int j = 0; j < m; ++j) {
      const float vj = cv[j];
      const int ij = ci[j];
      rank += (vj > v || (vj == v && ij < idx)) ? 1 : 0;
    }
    if (rank < k) { sv[rank] = v; si[rank] = idx; }
  }
  m = min(m, k);
  __syncthreads();
  const float top = sv[0];
  unsigned long long w = 0;
  if (tid < m) {
    w = (unsigned long long)(exp2f((sv[tid] - top) * c.inv_t2) * MASS_SCALE);
    if (w == 0) w = 1;
  }
  unsigned long long total;
  const unsigned long long incl = block_scan_incl(w, sh, total);
  __syncthreads();
  // top-p: shortest prefix whose mass reaches p * total ("include while the mass before it is < p")
  unsigned long long kept = total;
  if (top_p > 0.f && top_p < 1.f) {
    const unsigned long long want = (unsigned long long)(double(total) * double(top_p));
    if (tid == 0) sh.carry = total;
    __syncthreads();
    if (tid < m && incl >= want && incl - w < want) sh.carry = incl;  // exactly one thread
    __syncthreads();
    kept = sh.carry;
  }
  L.sv = sv; L.si = si; L.m = m; L.w = w; L.incl = incl; L.kept = kept;
}

// 53-bit uniform in [0, 1) from the stateless generator keyed by (seed, position).
__device__ __forceinline__ double uniform53(unsigned long long seed, unsigned long long position, uint32_t stream) {
  uint32_t rnd[4];
  Philox::gen(seed, position, stream, rnd);
  return double((((unsigned long long)rnd[0] << 32) | rnd[1]) >> 11) * (1.0 / 9007199254740992.0);
}
__device__ __forceinline__ double draw_uniform(const SampleParams& p, int row) {
  return uniform53(p.seeds ? p.seeds[row] : 0ull, (unsigned long long)(p.positions ? p.positions[row] : 0), 0x5a17u);
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(SampleParams p) {
  extern __shared__ unsigned long long priv[];  // [warps][256] private histograms; reused as the candidate list
  __shared__ SelectShared sh;
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ int cand_n;
  __shared__ float slice_bound;
  pdl_launch_dependents();
  pdl_wait();
  // Small batches: a thread-block cluster of C CTAs shares a row (one CTA scanning a 200k-entry row alone is bound by the
  // latency of its own loads); the other paths of the kernel are run by the cluster's first CTA.
  const unsigned C = samp_cluster_size(), crank = samp_cluster_rank();
  const int row = blockIdx.x / C, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = p.logits + size_t(row) * p.row_stride;
  const int n = p.vocab;
  const int k = p.top_k ? p.top_k[row] : 1;
  const float top_p = p.top_p ? p.top_p[row] : 0.f;
  const float temp = p.temperature ? p.temperature[row] : 1.f;
  const bool greedy = (k == 1 || temp <= 0.f);
  const bool small = !greedy && k > 1 && k < n && k <= SMALL_K;
  if (!small && crank != 0) return;      // uniform over the cluster: no cluster barrier is met on those paths

  float mx = 0.f;
  int arg = 0;
  if (!small) {
    // ---- maximum and its lowest index (greedy rows stop here; the full-vocabulary path needs the max)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int base = 0; base < n; base += 8 * blockDim.x) {   // 8 independent loads per thread and trip
      float vals[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < n ? x[i] : -INFINITY; }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i < n && (vals[u] > bv || (vals[u] == bv && i < bi))) { bv = vals[u]; bi = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < (blockDim.x >> 5) ? red_v[lane] : -INFINITY;
      bi = lane < (blockDim.x >> 5) ? red_i[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) { red_v[0] = bv; red_i[0] = bi; }
    }
    __syncthreads();
    mx = red_v[0];
    arg = red_i[0] == 0x7fffffff ? 0 : red_i[0];
    if (greedy || !(mx > -INFINITY)) {
      if (tid == 0) p.out[row] = arg;
      return;
    }
  }

  RowCtx c;
  c.x = x; c.n = n; c.mx = mx; c.inv_t2 = SAMP_LOG2E / temp;
  c.use_k = false; c.tk = 0; c.tk_idx = n;

  if (small) {
    // ---- top-k by count, then everything else on the k candidates
    SmallList L;
    small_list(c, sh, priv, &cand_n, k, top_p, L, C, crank, &slice_bound);
    if (crank != 0) return;
    unsigned long long target = (unsigned long long)(draw_uniform(p, row) * double(L.kept));
    if (target >= L.kept) target = L.kept - 1;
    if (tid < L.m && L.incl > target && L.incl - L.w <= target) p.out[row] = L.si[tid];
    return;
  }

  // ---- full-vocabulary path (no top-k, or k > SMALL_K)
  if (k > 1 && k < n) {
    radix_select<false>(c, sh, priv, (unsigned long long)k);
    const uint32_t T = sh.prefix;
    const unsigned long long need = sh.want, ties = sh.ties;
    __syncthreads();
    int cut = n;
    if (need < ties) cut = tie_index_cut<false>(c, sh, T, need, false);
    c.use_k = true; c.tk = T; c.tk_idx = cut;
    __syncthreads();
  }

  // final membership threshold (tp, tp_idx): starts as the top-k set, narrowed by top-p
  uint32_t tp = c.use_k ? c.tk : 0u;
  int tp_idx = c.use_k ? c.tk_idx : n;
  if (top_p > 0.f && top_p < 1.f) {
    unsigned long long z = 0;
    for (int base = 0; base < n; base += 8 * blockDim.x) {
      float vals[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < n ? x[i] : 0.f; }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = base + u * blockDim.x + tid;
        if (i < n && c.in_k(i, to_key(vals[u]))) z += c.mass(vals[u]);
      }
    }
    unsigned long long total;
    block_scan_incl(z, sh, total);
    __syncthreads();
    unsigned long long want = (unsigned long long)(double(total) * double(top_p));
    if (want < 1) want = 1;
    radix_select<true>(c, sh, priv, want);
    const uint32_t T = sh.prefix;
    const unsigned long long need = sh.want, ties = sh.ties;
    __syncthreads();
    int cut = n;
    if (need < ties) cut = tie_index_cut<true>(c, sh, T, need, true);
    __syncthreads();
    tp = T; tp_idx = cut;
  }

  // draw: prefix scan over kept masses in index order
  auto kept_mass_of = [&](int i, float v) -> unsigned long long {
    const uint32_t key = to_key(v);
    if (!c.in_k(i, key)) return 0ull;
    if (key > tp || (key == tp && i <= tp_idx)) { const unsigned long long m = c.mass(v); return m ? m : 1ull; }
    return 0ull;
  };
  auto kept_mass = [&](int i) -> unsigned long long {
    const float v = x[i];
    const uint32_t key = to_key(v);
    if (!c.in_k(i, key)) return 0ull;
    if (key > tp || (key == tp && i <= tp_idx)) { const unsigned long long m = c.mass(v); return m ? m : 1ull; }
    return 0ull;
  };
  unsigned long long z = 0;
  for (int base = 0; base < n; base += 8 * blockDim.x) {
    float vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < n ? x[i] : 0.f; }
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int i = base + u * blockDim.x + tid; if (i < n) z += kept_mass_of(i, vals[u]); }
  }
  unsigned long long zt;
  block_scan_incl(z, sh, zt);
  __syncthreads();
  unsigned long long target = (unsigned long long)(draw_uniform(p, row) * double(zt));
  if (target >= zt) target = zt - 1;

  if (tid == 0) { sh.carry = 0; sh.result = arg; }
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    const unsigned long long w = i < n ? kept_mass(i) : 0ull;
    unsigned long long total;
    const unsigned long long incl = block_scan_incl(w, sh, total);
    const unsigned long long carry = sh.carry;
    if (w && carry + incl > target && carry + incl - w <= target) sh.result = i;
    __syncthreads();
    const bool done = carry + total > target;
    if (tid == 0) sh.carry = carry + total;
    __syncthreads();
    if (done) break;
  }
  if (tid == 0) p.out[row] = sh.result;
}

// ------------------------------------------------------------------------------------ top-k scores
// Per row: the k largest entries (k <= 128), sorted descending (ties by lower index), written as
// values and indices.  mode 0: raw values; mode 1: log-softmax values plus add[row] (beam search:
// log-probabilities plus the running beam score, reference src/search.cpp:101-140).
constexpr int TOPK_MAX = 128;

struct TopKParams {
  const float* x; long long row_stride; int n, rows, k, mode;
  const float* add;
  float* out_vals; int32_t* out_idx;
};

__global__ void __launch_bounds__(SAMP_THREADS) topk_kernel(TopKParams p) {
  extern __shared__ unsigned long long priv[];
  __shared__ SelectShared sh;
  __shared__ float cand_v[TOPK_MAX];
  __shared__ int cand_i[TOPK_MAX];
  __shared__ int cand_n;
  __shared__ float red[32];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = p.x + size_t(row) * p.row_stride;
  const int n = p.n, k = min(p.k, n);

  // Every pass over the row issues UNR independent loads per thread and trip: a loop of single dependent loads costs one
  // L2 round trip per element and thread (measured: 201 us for 64 rows of 128256 before, against 36 us for the sampler).
  constexpr int UNR = 8;
  float mx = 0.f, lse = 0.f;
  if (p.mode == 1) {
    // log-softmax: row maximum and sum of exponentials in ONE pass (online rescaling)
    float s = 0.f;
    mx = -INFINITY;
    for (int base = 0; base < n; base += UNR * blockDim.x) {
      float vals[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < n ? x[i] : -INFINITY; }
      float bm = mx;
#pragma unroll
      for (int u = 0; u < UNR; ++u) bm = fmaxf(bm, vals[u]);
      if (bm > -INFINITY) {
        s *= __expf(mx - bm);
#pragma unroll
        for (int u = 0; u < UNR; ++u) s += __expf(vals[u] - bm);
        mx = bm;
      }
    }
    // combine (max, sum) pairs over the block
    float wm = warp_max(mx);
    s *= (mx > -INFINITY) ? __expf(mx - wm) : 0.f;
    s = warp_sum(s);
    __shared__ float red_s[32];
    if (lane == 0) { red[warp] = wm; red_s[warp] = s; }
    __syncthreads();
    if (warp == 0) {
      float m2 = lane < (blockDim.x >> 5) ? red[lane] : -INFINITY;
      float s2 = lane < (blockDim.x >> 5) ? red_s[lane] : 0.f;
      const float gm = warp_max(m2);
      s2 *= (m2 > -INFINITY) ? __expf(m2 - gm) : 0.f;
      s2 = warp_sum(s2);
      if (lane == 0) { red[0] = gm; red_s[0] = s2; }
    }
    __syncthreads();
    mx = red[0];
    lse = mx + __logf(red_s[0]);
    __syncthreads();
  }

  RowCtx c;
  c.x = x; c.n = n; c.mx = mx; c.inv_t2 = SAMP_LOG2E; c.use_k = false; c.tk = 0; c.tk_idx = n;
  uint32_t T = 0;
  int cut = n;
  if (k < n) {
    radix_select<false>(c, sh, priv, (unsigned long long)k);
    T = sh.prefix;
    const unsigned long long need = sh.want, ties = sh.ties;
    __syncthreads();
    if (need < ties) cut = tie_index_cut<false>(c, sh, T, need, false);
    __syncthreads();
  }
  if (tid == 0) cand_n = 0;
  __syncthreads();
  for (int base = 0; base < n; base += UNR * blockDim.x) {
    float vals[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < n ? x[i] : 0.f; }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int i = base + u * blockDim.x + tid;
      if (i >= n) continue;
      const uint32_t key = to_key(vals[u]);
      if (k >= n || key > T || (key == T && i <= cut)) {
        const int slot = atomicAdd(&cand_n, 1);
        if (slot < TOPK_MAX) { cand_v[slot] = vals[u]; cand_i[slot] = i; }
      }
    }
  }
  __syncthreads();
  const int m = min(cand_n, TOPK_MAX);
  // rank sort (m <= 128): position = number of candidates that come before this one
  if (tid < m) {
    const float v = cand_v[tid];
    const int idx = cand_i[tid];
    int rank = 0;
    for (int j = 0; j < m; ++j) {
      const float vj = cand_v[j];
      const int ij = cand_i[j];
      if (vj > v || (vj == v && ij < idx)) ++rank;
    }
    if (rank < k) {
      float outv = v;
      if (p.mode == 1) outv = v - lse + (p.add ? p.add[row] : 0.f);
      p.out_vals[size_t(row) * p.k + rank] = outv;
      p.out_idx[size_t(row) * p.k + rank] = idx;
    }
  }
}

// The same result for long rows, in two light passes: the candidate-list selection of the sampler (small_list: a bound from
// the per-thread maxima, then one filtered collection, with the exact radix select as its fall-back), optionally with the row
// split over the CTAs of a cluster.  mode 1 needs the row's log-sum-exp: each CTA reduces (max, sum of exponentials) over its
// slice in a pass of its own and deposits the pair in CTA 0's shared memory before the list is built.
__global__ void __launch_bounds__(SAMP_THREADS) topk_list_kernel(TopKParams p) {
  extern __shared__ unsigned long long priv[];
  __shared__ SelectShared sh;
  __shared__ int cand_n;
  __shared__ float slice_bound;
  __shared__ float part_m[8], part_s[8];
  __shared__ float red[32], red_s[32];
  const unsigned C = samp_cluster_size(), crank = samp_cluster_rank();
  const int row = blockIdx.x / int(C), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = p.x + size_t(row) * p.row_stride;
  const int n = p.n, k = p.k;
  if (p.mode == 1) {
    const int per = C > 1 ? ((n + int(C) - 1) / int(C) + 3) & ~3 : n;
    const int lo = min(n, int(crank) * per), hi = min(n, lo + per);
    float s = 0.f, mx = -INFINITY;
    for (int base = lo; base < hi; base += 8 * blockDim.x) {
      float vals[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { const int i = base + u * blockDim.x + tid; vals[u] = i < hi ? x[i] : -INFINITY; }
      float bm = mx;
#pragma unroll
      for (int u = 0; u < 8; ++u) bm = fmaxf(bm, vals[u]);
      if (bm > -INFINITY) {
        s *= __expf(mx - bm);
#pragma unroll
        for (int u = 0; u < 8; ++u) s += __expf(vals[u] - bm);
        mx = bm;
      }
    }
    if (C > 1) samp_cluster_sync();   // CTA 0 is running before anything is stored into its shared memory
    const float wm = warp_max(mx);
    s *= (mx > -INFINITY) ? __expf(mx - wm) : 0.f;
    s = warp_sum(s);
    if (lane == 0) { red[warp] = wm; red_s[warp] = s; }
    __syncthreads();
    if (warp == 0) {
      const float m2 = lane < (blockDim.x >> 5) ? red[lane] : -INFINITY;
      float s2 = lane < (blockDim.x >> 5) ? red_s[lane] : 0.f;
      const float gm = warp_max(m2);
      s2 *= (m2 > -INFINITY) ? __expf(m2 - gm) : 0.f;
      s2 = warp_sum(s2);
      if (lane == 0) {
        if (C > 1) {  // made visible to CTA 0 by the cluster barriers inside small_list
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(samp_dsmem(&part_m[crank], 0)), "f"(gm) : "memory");
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(samp_dsmem(&part_s[crank], 0)), "f"(s2) : "memory");
        } else {
          part_m[0] = gm; part_s[0] = s2;
        }
      }
    }
    __syncthreads();
  }
  RowCtx c;
  c.x = x; c.n = n; c.mx = 0.f; c.inv_t2 = SAMP_LOG2E; c.use_k = false; c.tk = 0; c.tk_idx = n;
  SmallList L;
  small_list(c, sh, priv, &cand_n, k, 0.f, L, C, crank, &slice_bound);
  if (crank != 0) return;
  float shift = 0.f;
  if (p.mode == 1) {
    float gm = -INFINITY, gs = 0.f;
    for (unsigned r = 0; r < C; ++r) gm = fmaxf(gm, part_m[r]);
    for (unsigned r = 0; r < C; ++r) gs += part_m[r] > -INFINITY ? part_s[r] * __expf(part_m[r] - gm) : 0.f;
    shift = (p.add ? p.add[row] : 0.f) - (gm + __logf(gs));
  }
  if (tid < L.m) {
    p.out_vals[size_t(row) * k + tid] = L.sv[tid] + shift;
    p.out_idx[size_t(row) * k + tid] = L.si[tid];
  }
}

// Beam merge: for each batch entry, the best 2*beams of its beams*(2*beams) candidates.
// in_vals / in_idx: [batch*beams, cand]; out: [batch, cand] scores, tokens, source beams.
__global__ void beam_merge_kernel(const float* in_vals, const int32_t* in_idx, int beams, int cand, float* out_scores,
                                  int32_t* out_tokens, int32_t* out_beams) {
  const int b = blockIdx.x;
  const int total = beams * cand;
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    const float v = in_vals[size_t(b) * total + e];
    int rank = 0;
    for (int j = 0; j < total; ++j) {
      const float vj = in_vals[size_t(b) * total + j];
      if (vj > v || (vj == v && j < e)) ++rank;
    }
    if (rank < cand) {
      out_scores[size_t(b) * cand + rank] = v;
      out_tokens[size_t(b) * cand + rank] = in_idx[size_t(b) * total + e];
      out_beams[size_t(b) * cand + rank] = e / cand;
    }
  }
}

// ------------------------------------------------------------------------------------ argmax rows
__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* logits, long long row_stride, int n, int32_t* out) {
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = logits + size_t(row) * row_stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int base = 0; base < n; base += 8 * blockDim.x) {   // 8 independent loads per thread and trip
    float vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x + tid;
      vals[u] = i < n ? x[i] : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + u * blockDim.x + tid;
      if (i < n && (vals[u] > bv || (vals[u] == bv && i < bi))) { bv = vals[u]; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? red_v[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

// ------------------------------------------------------------------------------------ speculative verify (greedy)
// target_argmax[K+1] vs draft[K]: accepted = length of the matching prefix; commit = accepted draft
// tokens followed by the target's token at the first mismatch (or the bonus token).  One thread.
__global__ void verify_greedy_kernel(const int32_t* draft, const int32_t* target_argmax, int k, int32_t* accepted, int32_t* commit) {
  if (threadIdx.x || blockIdx.x) return;
  int a = 0;
  while (a < k && draft[a] == target_argmax[a]) { commit[a] = draft[a]; ++a; }
  commit[a] = target_argmax[a];
  *accepted = a;
}

// ------------------------------------------------------------------------------------ speculative verify (sampled)
// Rejection sampling over K draft tokens in one launch (reference on the host: src/speculative_sampling.h:39-177).
// Block i < K: p = the target's sampled distribution of row i (temperature, top-k, top-p as in sample_kernel),
// q = the draft's distribution for that position (sparse list, or one-hot on the draft token when its list is
// empty: greedy draft, n-gram proposal).  It records accept_i = [u < min(1, p(x_i)/q(x_i))] and a token drawn
// from the residual max(0, p - q) renormalised (from p when the residual is empty).  Block K draws the bonus
// token from p_K with the same random stream the plain sampler would use at that position.  The last block
// to finish scans the decisions: accepted = first rejected position (K if none), commit = accepted drafts +
// the replacement / bonus token.  Rows need 1 < top_k <= 1024 (the sorted-list path).
struct VerifyParams {
  const float* logits; long long row_stride; int vocab, K;
  const int32_t* top_k; const float* top_p; const float* temperature;
  const unsigned long long* seeds; const int32_t* positions;   // per row
  const int32_t* draft;                                         // [K]
  const int32_t* q_idx; const float* q_prob; const int32_t* q_n; int q_stride;   // [K, q_stride]; q_n may be null (all one-hot)
  int32_t* accept; int32_t* resample;                           // [K + 1] scratch
  float* accept_prob;                                           // [K] (optional, statistics)
  unsigned int* done_count;                                     // zero before the first launch; the kernel resets it
  int32_t* accepted; int32_t* commit; int32_t* status;          // status: 1 = a row fell outside the supported range
};

__global__ void __launch_bounds__(SAMP_THREADS) verify_sampled_kernel(VerifyParams p) {
  extern __shared__ unsigned long long priv[];
  __shared__ SelectShared sh;
  __shared__ int cand_n;
  __shared__ double pt_sh;
  __shared__ int last_block;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int n = p.vocab, K = p.K;
  const int k = p.top_k ? p.top_k[row] : 0;
  const float top_p = p.top_p ? p.top_p[row] : 0.f;
  const float temp = p.temperature ? p.temperature[row] : 1.f;
  const unsigned long long seed = p.seeds ? p.seeds[row] : 0ull;
  const unsigned long long pos = (unsigned long long)(p.positions ? p.positions[row] : 0);
  const bool supported = k > 1 && k < n && k <= SMALL_K && temp > 0.f;
  if (!supported) {
    if (tid == 0) { atomicExch(p.status, 1); p.accept[row] = 0; p.resample[row] = 0; }
  } else {
    RowCtx c;
    c.x = p.logits + size_t(row) * p.row_stride; c.n = n; c.mx = 0.f; c.inv_t2 = SAMP_LOG2E / temp;
    c.use_k = false; c.tk = 0; c.tk_idx = n;
    SmallList L;
    small_list(c, sh, priv, &cand_n, k, top_p, L, 1u, 0u, nullptr);
    const bool in_p = tid < L.m && L.incl <= L.kept;   // entry belongs to the sampled distribution
    const bool bonus = row == K;
    const int x = bonus ? -1 : p.draft[row];
    const int qn = (bonus || !p.q_n) ? 0 : min(p.q_n[row], p.q_stride);
    const int32_t* qi = p.q_idx + size_t(bonus ? 0 : row) * p.q_stride;
    const float* qp = p.q_prob + size_t(bonus ? 0 : row) * p.q_stride;
    auto q_of = [&](int token) -> float {
      if (qn == 0) return token == x ? 1.f : 0.f;
      for (int j = 0; j < qn; ++j) if (qi[j] == token) return qp[j];
      return 0.f;
    };
    if (tid == 0) pt_sh = 0.0;
    __syncthreads();
    if (!bonus && in_p && L.si[tid] == x) pt_sh = double(L.w) / double(L.kept);
    __syncthreads();
    // residual mass of this thread's entry
    unsigned long long r = 0;
    if (in_p) {
      if (bonus) r = L.w;
      else {
        const double qq = double(q_of(L.si[tid])) * double(L.kept);
        r = double(L.w) > qq ? (unsigned long long)(double(L.w) - qq) : 0ull;
      }
    }
    unsigned long long rt;
    unsigned long long rincl = block_scan_incl(r, sh, rt);
    __syncthreads();
    if (rt == 0) {  // empty residual (p <= q everywhere): draw from p itself
      r = in_p ? L.w : 0ull;
      rincl = block_scan_incl(r, sh, rt);
      __syncthreads();
    }
    unsigned long long target = (unsigned long long)(uniform53(seed, pos, 0x5a17u) * double(rt));
    if (target >= rt) target = rt - 1;
    if (r && rincl > target && rincl - r <= target) p.resample[row] = L.si[tid];
    if (tid == 0) {
      if (bonus) {
        p.accept[row] = 0;
      } else {
        const float pt = float(pt_sh), qx = q_of(x);
        const float a = qx > 0.f ? fminf(1.f, pt / qx) : (pt > 0.f ? 1.f : 0.f);
        if (p.accept_prob) p.accept_prob[row] = a;
        p.accept[row] = uniform53(seed, pos, 0x5a18u) < double(a) ? 1 : 0;
      }
    }
  }
  // ---- the last block to finish scans the decisions
  __threadfence();
  __syncthreads();
  if (tid == 0) last_block = (atomicAdd(p.done_count, 1u) == unsigned(K)) ? 1 : 0;
  __syncthreads();
  if (last_block && tid == 0) {
    __threadfence();
    int a = 0;
    const volatile int32_t* acc = p.accept;
    const volatile int32_t* res = p.resample;
    while (a < K && acc[a]) { p.commit[a] = p.draft[a]; ++a; }
    p.commit[a] = res[a];
    *p.accepted = a;
    *p.done_count = 0;   // ready for the next launch (graph replay included)
  }
}

}  // namespace ogb

using namespace ogb;

OGB_API int ogb_sample(const float* logits, long long row_stride, int rows, int vocab, const int32_t* top_k, const float* top_p,
                       const float* temperature, const unsigned long long* seeds, const int32_t* positions, int32_t* out,
                       void* stream) {
  if (rows <= 0) return 0;
  SampleParams p{logits, row_stride, vocab, rows, top_k, top_p, temperature, seeds, positions, out};
  constexpr int kDyn = (SAMP_THREADS / 32) * 256 * 8;  // 64 KiB of per-warp histograms
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(sample_kernel, kDyn, configured)) return -3;
  // Rows per launch decide how many CTAs share a row: a cluster of 8 / 4 / 2 while all clusters fit the GPU in one wave.
  static const int sms = [] { int d = 0, n = 148; if (cudaGetDevice(&d) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d); return n; }();
  static const int cluster_env = [] { const char* e = getenv("OGB_SAMPLE_CLUSTER"); return e ? atoi(e) : -1; }();
  int C = rows * 8 <= sms ? 8 : (rows * 4 <= sms ? 4 : (rows * 2 <= sms ? 2 : 1));
  if (cluster_env >= 1 && cluster_env <= 8) C = cluster_env;
  if (vocab < 16384) C = 1;       // short rows: one CTA is already a few microseconds
  static const int pdl = [] { const char* e = getenv("OGB_PDL"); return (e && e[0] == '0') ? 0 : 1; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(rows) * unsigned(C));
  cfg.blockDim = dim3(SAMP_THREADS);
  cfg.dynamicSmemBytes = kDyn;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (C > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = unsigned(C); attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = unsigned(na);
  return cudaLaunchKernelEx(&cfg, sample_kernel, p) == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_argmax(const float* logits, long long row_stride, int rows, int vocab, int32_t* out, void* stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, SAMP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(logits, row_stride, vocab, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_topk(const float* x, long long row_stride, int rows, int n, int k, int mode, const float* add, float* out_vals,
                     int32_t* out_idx, void* stream) {
  if (rows <= 0) return 0;
  if (k < 1 || k > TOPK_MAX) return -1;
  TopKParams p{x, row_stride, n, rows, k, mode, add, out_vals, out_idx};
  constexpr int kDyn = (SAMP_THREADS / 32) * 256 * 8;
  if (k < n && n >= 4096) {
    // long rows: candidate-list kernel, a cluster of CTAs per row while all clusters fit the GPU in one wave
    static bool configured_list[OGB_MAX_DEVICES] = {};
    if (!set_max_dyn_smem(topk_list_kernel, kDyn, configured_list)) return -3;
    static const int sms = [] { int d = 0, v = 148; if (cudaGetDevice(&d) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d); return v; }();
    int C = rows * 8 <= sms ? 8 : (rows * 4 <= sms ? 4 : (rows * 2 <= sms ? 2 : 1));
    if (n < 16384) C = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(rows) * unsigned(C));
    cfg.blockDim = dim3(SAMP_THREADS);
    cfg.dynamicSmemBytes = kDyn;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = unsigned(C); attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, topk_list_kernel, p) == cudaSuccess ? 0 : -4;
  }
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(topk_kernel, kDyn, configured)) return -3;
  topk_kernel<<<rows, SAMP_THREADS, kDyn, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_beam_merge(const float* in_vals, const int32_t* in_idx, int batch, int beams, int cand, float* out_scores,
                           int32_t* out_tokens, int32_t* out_beams, void* stream) {
  if (batch <= 0) return 0;
  beam_merge_kernel<<<batch, 256, 0, static_cast<cudaStream_t>(stream)>>>(in_vals, in_idx, beams, cand, out_scores, out_tokens, out_beams);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_verify_greedy(const int32_t* draft, const int32_t* target_argmax, int k, int32_t* accepted, int32_t* commit, void* stream) {
  verify_greedy_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(draft, target_argmax, k, accepted, commit);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Sampled speculative verification of K draft tokens against K + 1 rows of target logits; see verify_sampled_kernel.
// scratch: (2 * (K + 1) + 1) int32 of device memory, zero before the first use (the kernel leaves it reusable).
OGB_API int ogb_verify_sampled(const float* logits, long long row_stride, int vocab, int K, const int32_t* top_k, const float* top_p,
                               const float* temperature, const unsigned long long* seeds, const int32_t* positions,
                               const int32_t* draft, const int32_t* q_idx, const float* q_prob, const int32_t* q_n, int q_stride,
                               int32_t* scratch, float* accept_prob, int32_t* accepted, int32_t* commit, int32_t* status, void* stream) {
  if (K < 0 || K > 64 || vocab <= 0) return -1;
  VerifyParams p{logits, row_stride, vocab, K, top_k, top_p, temperature, seeds, positions, draft, q_idx, q_prob, q_n, q_stride,
                 scratch, scratch + (K + 1), accept_prob, reinterpret_cast<unsigned int*>(scratch + 2 * (K + 1)), accepted, commit, status};
  constexpr int kDyn = (SAMP_THREADS / 32) * 256 * 8;
  static bool configured[OGB_MAX_DEVICES] = {};
  if (!set_max_dyn_smem(verify_sampled_kernel, kDyn, configured)) return -3;
  verify_sampled_kernel<<<K + 1, SAMP_THREADS, kDyn, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
