// Beam-search scorer and sequence bookkeeping on the device.
//
// One step of beam search, after the model's logits have been reduced to the best 2 * num_beams candidates of every batch
// entry (ogb_topk with log-softmax + running beam score, then ogb_beam_merge): choose the num_beams live continuations,
// move candidates that end in an end-of-sequence token into the entry's list of finished hypotheses (ranked by
// sum of log-probabilities / length ^ length_penalty), decide whether the entry is done (its num_beams-th finished
// hypothesis cannot be beaten any more, or early stopping), and append the new column to the token sequences - each new row
// a copy of the row it continues.  All of it runs in one launch, one CTA per batch entry; what goes back to the host
// is num_beams (token, source row) pairs per entry plus the count of entries still open, so that the paged key / value
// cache (whose block tables live on the host) can follow the reordering.  A second kernel adds the open beams as
// hypotheses when generation stops at the length limit.
//
// The rules are those of the host scorer (native/search.cpp: BeamScorer::Process / AddHypothesis / Finalize), which
// follows the reference's beam scorer (its CUDA form: src/cuda/beam_search_scorer_cuda.cu:79-176 for the scoring,
// :195-230 for the append of the new column to the sequences).
//
// Storage.  Sequences: two buffers [rows][max_length] that swap roles each step (a new row reads an old row).
// Hypotheses: per entry num_beams token slots [max_length] that never move; `hyp_order[rank]` names the slot of the
// rank-th best hypothesis, so an insertion shifts a few integers instead of token rows.
#include <cstdint>

#include "common.cuh"
#include "kernels.h"

namespace ogb {

constexpr int BEAM_MAX = 32;        // num_beams <= 32
constexpr int BEAM_MAX_EOS = 8;     // end-of-sequence ids
constexpr int BEAM_THREADS = 256;

struct BeamState {
  int32_t* seq[2];        // [rows][max_length]
  float* scores;          // [rows] running score of every live beam
  int32_t* hyp_tokens;    // [batch][num_beams][max_length]
  int32_t* hyp_len;       // [batch][num_beams] by slot
  float* hyp_score;       // [batch][num_beams] by slot
  int32_t* hyp_order;     // [batch][num_beams] rank -> slot
  int32_t* hyp_count;     // [batch]
  int32_t* done;          // [batch]
  int32_t* out;           // [2 * rows + 2]: next tokens, source rows, open entries, error flag
  int batch, num_beams, max_length, pad_token, early_stopping, n_eos;
  float length_penalty;
  int32_t eos[BEAM_MAX_EOS];
};

__device__ __forceinline__ bool beam_is_eos(const BeamState& st, int tok) {
  for (int i = 0; i < st.n_eos; ++i)
    if (st.eos[i] == tok) return true;
  return false;
}

// Thread 0 decides where a hypothesis of `len` tokens with `sum_logprobs` goes: returns the slot to fill (or -1 when it
// does not make the list) and updates order / count / score / length.
__device__ int beam_place_hypothesis(const BeamState& st, int b, int len, float sum_logprobs) {
  const int nb = st.num_beams;
  int32_t* order = st.hyp_order + b * nb;
  float* hscore = st.hyp_score + b * nb;
  int count = st.hyp_count[b];
  const float score = sum_logprobs / powf(float(len), st.length_penalty);
  if (count == nb && score <= hscore[order[nb - 1]]) return -1;
  int pos = 0;
  while (pos < count && !(score > hscore[order[pos]])) ++pos;
  int slot;
  if (count < nb) {
    slot = count;            // slots are handed out in order while the list grows
    ++count;
  } else {
    slot = order[nb - 1];    // the worst hypothesis gives up its slot
  }
  for (int i = count - 1; i > pos; --i) order[i] = order[i - 1];
  order[pos] = slot;
  hscore[slot] = score;
  st.hyp_len[b * nb + slot] = len;
  st.hyp_count[b] = count;
  return slot;
}

// cand_*: [batch][2 * num_beams], best first; scores include the running beam score.  `cur`: which sequence buffer holds
// the rows of length `len`.
__global__ void __launch_bounds__(BEAM_THREADS)
beam_step_kernel(const BeamState st, const float* __restrict__ cand_scores, const int32_t* __restrict__ cand_tokens,
                 const int32_t* __restrict__ cand_beams, int cur, int len) {
  const int b = blockIdx.x, nb = st.num_beams, cand = 2 * nb, L = st.max_length;
  __shared__ int s_tok[BEAM_MAX], s_row[BEAM_MAX];
  __shared__ float s_score[BEAM_MAX];
  __shared__ int s_slot, s_src, s_filled;
  const int32_t* old_seq = st.seq[cur];
  int32_t* new_seq = st.seq[cur ^ 1];
  const bool was_done = st.done[b] != 0;
  if (threadIdx.x == 0) s_filled = 0;
  __syncthreads();
  if (was_done) {
    if (threadIdx.x < nb) { s_tok[threadIdx.x] = st.pad_token; s_row[threadIdx.x] = b * nb; s_score[threadIdx.x] = 0.f; }
  } else {
    for (int j = 0; j < cand; ++j) {
      if (threadIdx.x == 0) {
        s_slot = -1;
        if (s_filled < nb) {
          const int tok = cand_tokens[b * cand + j];
          const float sc = cand_scores[b * cand + j];
          const int row = b * nb + cand_beams[b * cand + j];
          if (beam_is_eos(st, tok)) {
            if (j < nb) {            // an end-of-sequence candidate ranked below the beam width is dropped
              s_slot = beam_place_hypothesis(st, b, len, sc);
              s_src = row;
            }
          } else {
            s_tok[s_filled] = tok; s_row[s_filled] = row; s_score[s_filled] = sc;
            ++s_filled;
          }
        }
      }
      __syncthreads();
      if (s_slot >= 0) {
        int32_t* dst = st.hyp_tokens + (size_t(b) * nb + s_slot) * L;
        const int32_t* src = old_seq + size_t(s_src) * L;
        for (int i = threadIdx.x; i < len; i += blockDim.x) dst[i] = src[i];
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      if (s_filled != nb) {
        atomicMax(&st.out[2 * st.batch * nb + 1], 1);      // fewer than num_beams live candidates
        for (int k = s_filled; k < nb; ++k) { s_tok[k] = st.pad_token; s_row[k] = b * nb; s_score[k] = -1e9f; }
      }
      if (st.hyp_count[b] >= nb) {
        bool stop = true;
        if (!st.early_stopping) {
          float best = cand_scores[b * cand];
          for (int j = 1; j < cand; ++j) best = fmaxf(best, cand_scores[b * cand + j]);
          const float attainable = best / powf(float(len), st.length_penalty);
          const float worst = st.hyp_score[b * nb + st.hyp_order[b * nb + nb - 1]];
          if (worst < attainable) stop = false;
        }
        if (stop) {
          st.done[b] = 1;
          atomicSub(&st.out[2 * st.batch * nb], 1);
        }
      }
    }
  }
  __syncthreads();
  // the new column: row k continues old row s_row[k]
  if (threadIdx.x < nb) {
    const int r = b * nb + threadIdx.x;
    st.scores[r] = s_score[threadIdx.x];
    st.out[r] = s_tok[threadIdx.x];
    st.out[st.batch * nb + r] = s_row[threadIdx.x];
  }
  for (int k = 0; k < nb; ++k) {
    const int32_t* src = old_seq + size_t(s_row[k]) * L;
    int32_t* dst = new_seq + size_t(b * nb + k) * L;
    for (int i = threadIdx.x; i < len; i += blockDim.x) dst[i] = src[i];
    if (threadIdx.x == 0 && len < L) dst[len] = s_tok[k];
  }
}

// Generation stopped with entries still open: their live beams become hypotheses.
__global__ void __launch_bounds__(BEAM_THREADS) beam_finalize_kernel(const BeamState st, int cur, int len) {
  const int b = blockIdx.x, nb = st.num_beams, L = st.max_length;
  __shared__ int s_slot;
  if (st.done[b]) return;
  const int32_t* seq = st.seq[cur];
  for (int k = 0; k < nb; ++k) {
    const int row = b * nb + k;
    if (threadIdx.x == 0) s_slot = beam_place_hypothesis(st, b, len, st.scores[row]);
    __syncthreads();
    if (s_slot >= 0) {
      int32_t* dst = st.hyp_tokens + (size_t(b) * nb + s_slot) * L;
      const int32_t* src = seq + size_t(row) * L;
      for (int i = threadIdx.x; i < len; i += blockDim.x) dst[i] = src[i];
    }
    __syncthreads();
  }
}

}  // namespace ogb

using namespace ogb;

static bool FillState(BeamState& st, void* seq0, void* seq1, void* scores, void* hyp_tokens, void* hyp_len, void* hyp_score, void* hyp_order,
                      void* hyp_count, void* done, void* out, int batch, int num_beams, int max_length, int pad_token, int early_stopping,
                      float length_penalty, const int32_t* eos, int n_eos) {
  if (batch <= 0 || num_beams < 1 || num_beams > BEAM_MAX || max_length <= 0 || n_eos < 0 || n_eos > BEAM_MAX_EOS) return false;
  st.seq[0] = static_cast<int32_t*>(seq0); st.seq[1] = static_cast<int32_t*>(seq1);
  st.scores = static_cast<float*>(scores);
  st.hyp_tokens = static_cast<int32_t*>(hyp_tokens); st.hyp_len = static_cast<int32_t*>(hyp_len);
  st.hyp_score = static_cast<float*>(hyp_score); st.hyp_order = static_cast<int32_t*>(hyp_order);
  st.hyp_count = static_cast<int32_t*>(hyp_count); st.done = static_cast<int32_t*>(done); st.out = static_cast<int32_t*>(out);
  st.batch = batch; st.num_beams = num_beams; st.max_length = max_length; st.pad_token = pad_token; st.early_stopping = early_stopping;
  st.length_penalty = length_penalty; st.n_eos = n_eos;
  for (int i = 0; i < n_eos; ++i) st.eos[i] = eos[i];
  return true;
}

// One beam-search step on the device.  Buffers (all device memory, owned by the caller): seq0 / seq1 int32 [rows][max_length]
// (`cur` names the one that holds the current rows of `len` tokens; the other receives the rows of len + 1), scores fp32
// [rows], hyp_tokens int32 [batch][num_beams][max_length], hyp_len int32 / hyp_score fp32 / hyp_order int32
// [batch][num_beams], hyp_count / done int32 [batch], out int32 [2 * rows + 2] = next tokens, source rows, number of
// entries still open (initialised to batch by the caller), error flag (1: an entry had fewer than num_beams candidates
// that do not end a sequence).  eos: host array of up to 8 end-of-sequence ids.
OGB_API int ogb_beam_scorer_step(const float* cand_scores, const int32_t* cand_tokens, const int32_t* cand_beams, void* seq0, void* seq1,
                                 int cur, int len, void* scores, void* hyp_tokens, void* hyp_len, void* hyp_score, void* hyp_order,
                                 void* hyp_count, void* done, void* out, int batch, int num_beams, int max_length, int pad_token,
                                 int early_stopping, float length_penalty, const int32_t* eos, int n_eos, void* stream) {
  BeamState st;
  if (!FillState(st, seq0, seq1, scores, hyp_tokens, hyp_len, hyp_score, hyp_order, hyp_count, done, out, batch, num_beams, max_length,
                 pad_token, early_stopping, length_penalty, eos, n_eos))
    return -1;
  if (len < 1 || len > max_length || (cur != 0 && cur != 1)) return -1;
  beam_step_kernel<<<batch, BEAM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(st, cand_scores, cand_tokens, cand_beams, cur, len);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

OGB_API int ogb_beam_scorer_finalize(void* seq0, void* seq1, int cur, int len, void* scores, void* hyp_tokens, void* hyp_len, void* hyp_score,
                                     void* hyp_order, void* hyp_count, void* done, void* out, int batch, int num_beams, int max_length,
                                     int pad_token, int early_stopping, float length_penalty, const int32_t* eos, int n_eos, void* stream) {
  BeamState st;
  if (!FillState(st, seq0, seq1, scores, hyp_tokens, hyp_len, hyp_score, hyp_order, hyp_count, done, out, batch, num_beams, max_length,
                 pad_token, early_stopping, length_penalty, eos, n_eos))
    return -1;
  if (len < 1 || len > max_length || (cur != 0 && cur != 1)) return -1;
  beam_finalize_kernel<<<batch, BEAM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(st, cur, len);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
