// C entry points around the reference's own CUDA kernels (top-k with its online algorithm selection, beam-search top-k, grammar
// mask application), so that benchmark/benchmark_tail_kernels.py can time them on the same GPU as this framework's kernels.
// The reference sources are compiled unmodified from the reference tree by baseline/build_ref_kernels.py; this file only
// forwards calls (reference entry points: src/cuda/cuda_topk.h RunTopK, src/beam_search_topk.h BeamSearchTopK,
// src/cuda/model_kernels.cu LaunchAddLogitsMask).
#include <cuda_runtime.h>
#include <stdint.h>

#include "cuda_topk.h"

namespace Generators {
namespace cuda {
void BeamSearchTopK(const float* input, int32_t batch_size, int32_t num_beams, int32_t vocab_size, int32_t k, float* tmp_values_1st_stage,
                    int32_t* tmp_indices_1st_stage, float* tmp_values_2nd_stage, int32_t* tmp_indices_2nd_stage, float* output_values,
                    int32_t* output_tokens, int32_t* output_indices, cudaStream_t stream);
void LaunchAddLogitsMask(float* batch_logits, int batch_beam_size, int vocab_size, const uint32_t* logits_mask, cudaStream_t stream);
}  // namespace cuda
}  // namespace Generators

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void* ref_topk_create(int batch, int vocab, void* stream) {
  try {
    return new Generators::cuda::TopkData(batch, vocab, static_cast<cudaStream_t>(stream));
  } catch (...) {
    return nullptr;
  }
}

REF_API void ref_topk_destroy(void* h) { delete static_cast<Generators::cuda::TopkData*>(h); }

// Runs the reference's dispatcher (it benchmarks its algorithms on the first call of a shape and caches the winner).
// Returns 0, or -1 when the reference threw.  out_scores / out_indices / out_stride describe where its result lies.
REF_API int ref_topk_run(void* h, const float* scores, int vocab, int batch, int k, void* stream, const float** out_scores,
                         const int** out_indices, int* out_stride) {
  auto* d = static_cast<Generators::cuda::TopkData*>(h);
  try {
    Generators::cuda::RunTopK(d, static_cast<cudaStream_t>(stream), scores, vocab, batch, k);
  } catch (...) {
    return -1;
  }
  if (out_scores) *out_scores = d->topk_scores;
  if (out_indices) *out_indices = d->topk_indices;
  if (out_stride) *out_stride = d->topk_stride;
  return 0;
}

// tmp: batch * beams * 129 * beams * 2 * 2 floats (the sizing of src/cuda/search_cuda.cpp:66-68)
REF_API int ref_beam_topk(const float* log_probs, int batch, int beams, int vocab, int k, float* tmp, float* out_values, int32_t* out_tokens,
                          int32_t* out_indices, void* stream) {
  const size_t candidate_count = size_t(batch) * beams * 2 * beams, parts = 128;
  float* v1 = tmp;
  int32_t* i1 = reinterpret_cast<int32_t*>(v1 + candidate_count * parts);
  float* v2 = reinterpret_cast<float*>(i1 + candidate_count * parts);
  int32_t* i2 = reinterpret_cast<int32_t*>(v2 + candidate_count);
  try {
    Generators::cuda::BeamSearchTopK(log_probs, batch, beams, vocab, k, v1, i1, v2, i2, out_values, out_tokens, out_indices,
                                     static_cast<cudaStream_t>(stream));
  } catch (...) {
    return -1;
  }
  return 0;
}

REF_API int ref_add_logits_mask(float* logits, int rows, int vocab, const uint32_t* mask, void* stream) {
  try {
    Generators::cuda::LaunchAddLogitsMask(logits, rows, vocab, mask, static_cast<cudaStream_t>(stream));
  } catch (...) {
    return -1;
  }
  return 0;
}
