// Continuous-batching engine core: requests, paged KV block accounting, decode-first scheduling
// and the transactional step (plan -> reserve -> pack -> [execute on GPU] -> commit | abort).
//
// Contracts follow the reference engine (docs/paged_attention_engine.md; src/engine/engine.cpp:227-451,
// scheduler.cpp:145-275, decode_first_scheduler_policy.cpp:11-60, paged_cache_reservation.cpp:47-255,
// request.cpp:38-499, block.cpp):
//   * request states Unassigned -> Assigned -> Active -> TurnComplete -> (Continue -> Assigned) | Closed;
//   * the cache holds tokens [0, N), the request holds [0, N+1): token N is the next model input;
//   * a generated EOS is neither appended nor returned; max_length is cumulative across turns;
//   * residents are planned before waiting requests, decodes before prefills, every selected request
//     gets one token before prefills share the rest of max_scheduled_tokens;
//   * block reservation for a step is all-or-nothing per request; admission reserves the whole prompt;
//   * every block is in exactly one of {free, reserved by the open step, committed to a request};
//   * a retryable failure restores every request and releases the reservation; a fatal one marks the
//     engine unhealthy.
//
// What differs by design: the model itself runs outside (torch + CUDA kernels); this core writes the
// packed step inputs (token ids, positions, cu_seqlens, block tables, slot mapping, per-row sampling
// parameters) straight into caller-owned pinned host buffers so that one H2D copy feeds a whole step,
// and sampling parameters travel as per-row arrays instead of bucketing rows by (k, p, T).
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

namespace ogb::engine {

// ----------------------------------------------------------------------------------- block pool
class BlockPool {
 public:
  explicit BlockPool(int num_blocks);
  int Total() const { return int(state_.size()); }
  int FreeCount() const { return int(free_.size()); }
  // All-or-nothing: appends n block ids to `out` or returns false and leaves the pool untouched.
  bool Reserve(int n, std::vector<int>& out);
  void Commit(int id);   // reserved -> committed
  void Release(int id);  // reserved -> free
  void Free(int id);     // committed -> free; throws on a block that is not committed
  enum class State : uint8_t { kFree, kReserved, kCommitted };
  State StateOf(int id) const { return state_.at(size_t(id)); }

 private:
  std::vector<State> state_;
  std::vector<int> free_;  // kept sorted descending so the lowest id is handed out first
};

// ----------------------------------------------------------------------------------- requests
enum class RequestStatus { kUnassigned, kAssigned, kActive, kTurnComplete, kClosed };
const char* ToString(RequestStatus s);

struct SamplingArgs {
  // Resolved per-request arguments (reference: src/engine/scheduled_requests.cpp:18-30):
  // greedy -> {k=1, p=0, T=1}; top-k only -> {k, 1, T}; top-p only -> {-1, p, T}.
  int top_k{1};
  float top_p{0.f};
  float temperature{1.f};
};

struct RequestOptions {
  int max_length{0};
  int min_length{0};
  bool do_sample{false};
  int top_k{50};
  float top_p{0.f};
  float temperature{1.f};
  float repetition_penalty{1.f};
  int no_repeat_ngram_size{0};
  int random_seed{-1};
  int chunk_size{0};  // 0 = no per-request prefill cap
  int num_beams{1};
  int batch_size{1};
  SamplingArgs Resolve() const;
};

class Request {
 public:
  Request(uint64_t id, RequestOptions opt, std::vector<int32_t> eos_ids);
  uint64_t Id() const { return id_; }
  RequestStatus Status() const { return status_; }
  const RequestOptions& Options() const { return opt_; }
  const std::vector<int32_t>& Tokens() const { return tokens_; }
  int Processed() const { return processed_; }
  int Pending() const { return int(tokens_.size()) - processed_; }
  bool IsPrefill() const { return prefill_; }
  bool HasUnseen() const { return !unseen_.empty(); }
  int32_t PopUnseen();
  bool TurnComplete() const { return status_ == RequestStatus::kTurnComplete; }
  uint64_t Seed() const { return seed_; }

  void AddTokens(const int32_t* ids, size_t n);      // only while Unassigned
  void ContinueWith(const int32_t* ids, size_t n, int new_max_length = 0);   // only while TurnComplete; > 0: the limit from now on
  // Speculative decoding: stages up to n proposed continuation tokens behind the pending token of a decoding request.  The
  // next step then feeds [pending token, drafts...] (1 + n rows whose logits verify the proposal) and is closed with
  // EngineCore::CommitSpeculative.  Returns how many were staged (clipped so that the accepted tokens plus the correction or
  // bonus token stay below max_length; 0 for a request that is not decoding with exactly one pending token).
  int SetDraft(const int32_t* ids, size_t n);
  int DraftCount() const { return draft_; }
  const std::vector<int>& Blocks() const { return blocks_; }
  const std::vector<int>& WindowBlocks() const { return window_blocks_; }

 private:
  friend class EngineCore;
  struct Saved {
    size_t token_count;
    int processed;
    size_t unseen;
    RequestStatus status;
    bool prefill;
    size_t block_count, window_block_count;
  };
  uint64_t id_;
  RequestOptions opt_;
  std::vector<int32_t> eos_ids_;
  RequestStatus status_{RequestStatus::kUnassigned};
  std::vector<int32_t> tokens_;
  int processed_{0};
  bool prefill_{true};
  std::deque<int32_t> unseen_;
  std::vector<int> blocks_;         // committed blocks of the full-attention layers
  std::vector<int> window_blocks_;  // ring blocks of the sliding-window layers
  uint64_t seed_;
  int draft_{0};                    // trailing tokens of tokens_ that are an unverified proposal
  bool resident_{false};
  std::optional<Saved> saved_;
};

// ----------------------------------------------------------------------------------- step plan
enum class StepOutcome {
  kNoWork, kCapacityDeferred, kUnserviceableRequest, kCommitted, kRetryableBatchAbort,
  kExecutionCapacityExceeded, kExecutionContractFailure, kFatalExecutionFailure, kPlanned
};
const char* ToString(StepOutcome o);

enum class FailureKind { kRetryableBeforeExecution, kRetryableDuringExecution, kCapacityExceeded, kFatal, kPostProcessing };

struct PlanEntry {
  std::shared_ptr<Request> request;
  int num_tokens{};        // tokens fed this step
  int packed_offset{};     // offset into the flat token array
  int logits_row{};        // row of the packed output that predicts the next token
  int processed_before{};  // KV slots already committed
  bool is_prefill{};
  bool samples{};          // true when this step consumes the request's last pending token
  bool newly_admitted{};
};

struct StepPlan {
  StepOutcome outcome{StepOutcome::kNoWork};
  std::vector<PlanEntry> entries;
  int token_count{0};
  int max_query_len{0};
  int max_kv_len{0};
  int block_table_columns{0};  // exact number of columns needed
  bool graph_eligible{false};  // every entry is a 1-token decode
  // Decode look-ahead (EngineOptions::lookahead): the executor may enqueue the step after this one before this step's
  // tokens reach the host.  lookahead_ok: every entry is a 1-token decode that stays below its max_length and owns the
  // block its next position falls in.  signature identifies (request, position) of every entry in order;
  // next_signature is the signature the following plan has if the same requests simply advance by one token.
  bool lookahead_ok{false};
  uint64_t signature{0}, next_signature{0};
  std::vector<std::shared_ptr<Request>> unserviceable;
  int deferred{0};
};

struct EngineOptions {
  int block_size{256};
  int num_blocks{0};
  int max_batch_size{16};
  int max_scheduled_tokens{2048};
  bool static_batching{false};  // fixed batches: up to 4 waiting requests (then 2, then 1) are admitted together with all the
                                // blocks their max_length needs, and only once the batch before them has finished
  int lookahead{0};           // decode entries also reserve the block of their next `lookahead` positions
  bool lookahead_execution{true};  // false: the reservation above serves speculative drafts; plans never report lookahead_ok
  int window_size{0};         // > 0 enables the sliding-window ring pool
  int num_window_blocks{0};   // blocks in the windowed pool
  int vocab_size{0};
  int pad_token_id{0};
  std::vector<int32_t> eos_ids;
};

struct TransactionMetrics {
  uint64_t steps_committed{}, steps_aborted{}, steps_deferred{}, requests_admitted{}, requests_completed{},
      tokens_scheduled{}, tokens_generated{}, unserviceable{};
};

// Pointers into caller-owned (pinned) host memory; capacities are in elements.
struct PackBuffers {
  int32_t* input_ids{};       // [max tokens]
  int32_t* positions{};       // [max tokens]   absolute position of each token
  int32_t* token_row{};       // [max tokens]   batch row of each token
  int32_t* slot_mapping{};    // [max tokens]   block_id * block_size + offset (full-attention pool)
  int32_t* slot_mapping_w{};  // [max tokens]   same for the windowed pool (may be null)
  int32_t* cu_seqlens{};      // [B + 1]
  int32_t* past_lens{};       // [B]
  int32_t* logits_rows{};     // [B]
  int32_t* block_table{};     // [B, table_columns]
  int32_t* block_table_w{};   // [B, table_columns] (may be null)
  int32_t* top_k{};           // [B]
  float* top_p{};             // [B]
  float* temperature{};       // [B]
  uint64_t* seeds{};          // [B]
  int32_t* sample_pos{};      // [B]  sequence position the sampled token will occupy (RNG counter)
  int max_tokens{}, max_batch{}, table_columns{};
};

class EngineCore {
 public:
  explicit EngineCore(EngineOptions opt);

  std::shared_ptr<Request> CreateRequest(RequestOptions opt);
  void AddRequest(const std::shared_ptr<Request>& r);
  void RemoveRequest(const std::shared_ptr<Request>& r);
  bool HasPendingRequests() const;
  bool Healthy() const { return healthy_; }

  // P1 + P2 + P3: choose requests, reserve blocks, checkpoint.  When outcome == kPlanned a
  // transaction is open and must be closed with Commit or Abort.
  const StepPlan& Plan();
  // Writes the packed inputs of the open plan. table_columns must be >= plan.block_table_columns.
  void Pack(const PackBuffers& buf) const;
  // P5 + P6: tokens[i] is the sampled token of entry i (ignored where !entry.samples).
  StepOutcome Commit(const int32_t* tokens, size_t n);
  // The same for a step with staged drafts: accepted[i] of entry i's drafts were verified (0 for entries without drafts) and
  // tokens[i] is the token that follows them (the target's correction at the first rejection, its bonus token when every draft
  // was accepted, the ordinary sampled token without drafts).  The cache keeps the accepted drafts' slots; rejected drafts
  // leave the sequence.  A draft that is an end-of-sequence token ends the turn there.
  StepOutcome CommitSpeculative(const int32_t* accepted, const int32_t* tokens, size_t n);
  StepOutcome Abort(FailureKind kind, const std::string& what);
  bool TransactionOpen() const { return open_; }

  std::shared_ptr<Request> NextReady();  // a request with unseen tokens or a newly completed turn
  const TransactionMetrics& Metrics() const { return metrics_; }
  const EngineOptions& Options() const { return opt_; }
  int FreeBlocks() const { return pool_.FreeCount(); }
  int FreeWindowBlocks() const { return wpool_ ? wpool_->FreeCount() : 0; }
  int RingBlocksPerRequest() const { return ring_blocks_; }

  // Throws std::logic_error describing the first violated invariant (block ownership, counters).
  void CheckInvariants() const;

 private:
  void ReleaseRequestBlocks(Request& r);
  int BlocksFor(int slots) const { return (slots + opt_.block_size - 1) / opt_.block_size; }

  EngineOptions opt_;
  BlockPool pool_;
  std::unique_ptr<BlockPool> wpool_;
  int ring_blocks_{0};
  std::vector<std::shared_ptr<Request>> requests_;  // admission order
  std::deque<std::shared_ptr<Request>> ready_;
  StepPlan plan_;
  struct Reserved { std::vector<int> blocks, wblocks; };
  std::vector<Reserved> reserved_;  // parallel to plan_.entries
  bool open_{false};
  bool healthy_{true};
  uint64_t next_id_{1};
  TransactionMetrics metrics_;
};

}  // namespace ogb::engine
