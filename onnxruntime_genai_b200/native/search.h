// Token search state: sequences, EOS bookkeeping, greedy / sampled / beam selection.
//
// Behaviour mirrors the reference's Search family (src/search.h:31-271, src/search.cpp:101-278,
// src/beam_search_scorer.cpp:19-196): one int32 sequence buffer of [batch*beams, max_length]; a
// batch entry that produced EOS keeps emitting pad; generation ends when every entry is finished
// or max_length is reached; beams keep 2*num_beams candidates per batch entry and rank finished
// hypotheses by sum_logprobs / len^length_penalty.
//
// The same object serves two scoring devices: the host path (SelectTop / Sample* read fp32 logits
// set with SetLogits) and the device path (the GPU sampler or beam kernel picks tokens, the host
// calls CommitTokens / CommitBeamStep to keep sequences and EOS state in sync).
#pragma once
#include <cstdint>
#include <memory>
#include <random>
#include <vector>

#include "sampling.h"

namespace ogb {

struct SearchParams {
  int batch_size{1};
  int num_beams{1};
  int num_return_sequences{1};
  int max_length{0};
  int min_length{0};
  int vocab_size{0};
  int pad_token_id{0};
  std::vector<int32_t> eos_token_ids;
  float repetition_penalty{1.f};
  int no_repeat_ngram_size{0};
  float length_penalty{1.f};
  bool early_stopping{true};
  int random_seed{-1};
  int BatchBeam() const { return batch_size * num_beams; }
};

class Sequences {
 public:
  Sequences(int batch_beam, int max_length);
  int Length() const { return length_; }
  int Rows() const { return rows_; }
  const int32_t* Row(int r) const { return cur_.data() + size_t(r) * max_length_; }
  int32_t* Row(int r) { return cur_.data() + size_t(r) * max_length_; }
  void AppendPrompt(const int32_t* ids, int batch, int len, int num_beams);  // first call may expand beams
  void AppendColumn(const int32_t* tokens);                                  // one token per row
  void AppendBeamColumn(const int32_t* beam_src_rows, const int32_t* tokens); // reorder rows then append
  void DropLast(int new_length);                                              // rewind
  int32_t Last(int r) const { return Row(r)[length_ - 1]; }

 private:
  int rows_, max_length_, length_{0};
  std::vector<int32_t> cur_, alt_;
};

struct BeamHypothesis {
  std::vector<int32_t> tokens;
  float score{};
};

class BeamScorer {
 public:
  explicit BeamScorer(const SearchParams& p);
  // cand_* hold 2*num_beams candidates per batch entry, best first.  Fills next_* (num_beams per
  // batch entry) and moves finished candidates into the hypothesis lists.
  void Process(const Sequences& seq, const float* cand_scores, const int32_t* cand_tokens, const int32_t* cand_beams);
  void Finalize(const Sequences& seq);
  bool Done() const { return open_batches_ == 0; }
  const std::vector<float>& NextScores() const { return next_scores_; }
  const std::vector<int32_t>& NextTokens() const { return next_tokens_; }
  const std::vector<int32_t>& NextRows() const { return next_rows_; }
  // Ranked finished hypothesis `rank` (0 = best) of batch entry b; valid after Finalize.
  const BeamHypothesis& Hypothesis(int b, int rank) const;

 private:
  struct PerBatch {
    std::vector<BeamHypothesis> best;  // descending score, at most num_beams
    bool done{false};
  };
  void AddHypothesis(PerBatch& pb, const int32_t* toks, int len, float sum_logprobs);
  SearchParams p_;
  std::vector<PerBatch> per_batch_;
  std::vector<float> next_scores_;
  std::vector<int32_t> next_tokens_, next_rows_;
  int open_batches_;
  bool finalized_{false};
};

// Snapshot of everything a step may change; restoring it makes the step a no-op.
struct SearchCheckpoint {
  int length{};
  bool done{};
  int open_count{};
  std::vector<uint8_t> eos_seen;
  std::vector<int32_t> next_tokens;
  std::mt19937 rng;
};

class Search {
 public:
  explicit Search(const SearchParams& p);
  virtual ~Search() = default;

  const SearchParams& Params() const { return p_; }
  Sequences& Seqs() { return seq_; }
  int Length() const { return seq_.Length(); }
  bool IsDone() const { return done_; }
  const std::vector<int32_t>& NextTokens() const { return next_tokens_; }

  void AppendTokens(const int32_t* ids, int batch, int len);
  void RewindTo(int length);

  // Host scoring path.  `logits` is [batch*beams, vocab] fp32 and is modified in place.
  void SetLogits(float* logits) { logits_ = logits; }
  void ApplyMinLength();
  void ApplyRepetitionPenalty();
  void ApplyNoRepeatNgram();
  virtual void SelectTop();
  virtual void SampleTopK(int k, float temperature);
  virtual void SampleTopP(float p, float temperature);
  virtual void SampleTopKTopP(int k, float p, float temperature);

  // Device scoring path: tokens chosen elsewhere; applies pad-after-EOS, EOS accounting, append.
  virtual void CommitTokens(const int32_t* tokens);

  virtual bool IsBeam() const { return false; }
  SearchCheckpoint Save() const;
  void Restore(const SearchCheckpoint& c);
  std::mt19937& Rng() { return rng_; }

 protected:
  void Sample(int k, float p, float t);
  void FinishStep();
  SearchParams p_;
  Sequences seq_;
  float* logits_{nullptr};
  std::vector<int32_t> next_tokens_;
  std::vector<uint8_t> eos_seen_;
  int open_count_;
  bool done_{false};
  std::mt19937 rng_;
  std::vector<uint8_t> seen_scratch_;
  std::vector<int32_t> idx_scratch_;
};

class BeamSearch : public Search {
 public:
  explicit BeamSearch(const SearchParams& p);
  bool IsBeam() const override { return true; }
  void SelectTop() override;
  void SampleTopK(int, float) override { throw std::runtime_error("sampling is not supported with beam search"); }
  void SampleTopP(float, float) override { throw std::runtime_error("sampling is not supported with beam search"); }
  void SampleTopKTopP(int, float, float) override { throw std::runtime_error("sampling is not supported with beam search"); }
  void CommitTokens(const int32_t*) override { throw std::runtime_error("use CommitBeamStep with beam search"); }
  // Device path: 2*num_beams candidates per batch entry (scores already include the running beam score).
  void CommitBeamStep(const float* cand_scores, const int32_t* cand_tokens, const int32_t* cand_beams);
  // Device scorer path: the step was scored on the device; append the column (new row r continues old row rows[r]) and take
  // over its verdict.  The host scorer is not consulted; SetHypothesis supplies the ranked results at the end.
  void CommitBeamResult(const int32_t* tokens, const int32_t* rows, bool all_done);
  void SetHypothesis(int batch, int rank, const int32_t* tokens, int len, float score);
  const std::vector<int32_t>& NextRows() const { return device_scored_ ? device_rows_ : scorer_.NextRows(); }  // source row per new row
  const std::vector<float>& BeamScores() const { return scorer_.NextScores(); }
  void Finalize();
  const BeamHypothesis& Hypothesis(int batch, int rank) const;

 private:
  BeamScorer scorer_;
  bool finalized_{false};
  std::vector<int32_t> order_;
  bool device_scored_{false};
  std::vector<int32_t> device_rows_;
  std::vector<std::vector<BeamHypothesis>> device_hyps_;   // [batch][rank], filled by SetHypothesis
};

std::unique_ptr<Search> MakeSearch(const SearchParams& p);

}  // namespace ogb
