#include "engine_core.h"

#include <algorithm>
#include <random>
#include <stdexcept>

namespace ogb::engine {

// ----------------------------------------------------------------------------------- BlockPool
BlockPool::BlockPool(int n) : state_(size_t(n), State::kFree) {
  free_.reserve(size_t(n));
  for (int i = n - 1; i >= 0; --i) free_.push_back(i);
}

bool BlockPool::Reserve(int n, std::vector<int>& out) {
  if (n < 0) throw std::invalid_argument("BlockPool::Reserve: negative count");
  if (n > int(free_.size())) return false;
  for (int i = 0; i < n; ++i) {
    int id = free_.back();
    free_.pop_back();
    state_[size_t(id)] = State::kReserved;
    out.push_back(id);
  }
  return true;
}

void BlockPool::Commit(int id) {
  if (id < 0 || id >= Total() || state_[size_t(id)] != State::kReserved)
    throw std::logic_error("BlockPool::Commit: block " + std::to_string(id) + " is not reserved");
  state_[size_t(id)] = State::kCommitted;
}

static void InsertFree(std::vector<int>& free_list, int id) {
  // keep descending order so that back() is the lowest id
  auto it = std::lower_bound(free_list.begin(), free_list.end(), id, std::greater<int>());
  free_list.insert(it, id);
}

void BlockPool::Release(int id) {
  if (id < 0 || id >= Total() || state_[size_t(id)] != State::kReserved)
    throw std::logic_error("BlockPool::Release: block " + std::to_string(id) + " is not reserved");
  state_[size_t(id)] = State::kFree;
  InsertFree(free_, id);
}

void BlockPool::Free(int id) {
  if (id < 0 || id >= Total() || state_[size_t(id)] != State::kCommitted)
    throw std::logic_error("BlockPool::Free: block " + std::to_string(id) + " is not committed");
  state_[size_t(id)] = State::kFree;
  InsertFree(free_, id);
}

// ----------------------------------------------------------------------------------- strings
const char* ToString(RequestStatus s) {
  switch (s) {
    case RequestStatus::kUnassigned: return "Unassigned";
    case RequestStatus::kAssigned: return "Assigned";
    case RequestStatus::kActive: return "Active";
    case RequestStatus::kTurnComplete: return "TurnComplete";
    case RequestStatus::kClosed: return "Closed";
  }
  return "?";
}
const char* ToString(StepOutcome o) {
  switch (o) {
    case StepOutcome::kNoWork: return "NoWork";
    case StepOutcome::kCapacityDeferred: return "CapacityDeferred";
    case StepOutcome::kUnserviceableRequest: return "UnserviceableRequest";
    case StepOutcome::kCommitted: return "Committed";
    case StepOutcome::kRetryableBatchAbort: return "RetryableBatchAbort";
    case StepOutcome::kExecutionCapacityExceeded: return "ExecutionCapacityExceeded";
    case StepOutcome::kExecutionContractFailure: return "ExecutionContractFailure";
    case StepOutcome::kFatalExecutionFailure: return "FatalExecutionFailure";
    case StepOutcome::kPlanned: return "Planned";
  }
  return "?";
}

// ----------------------------------------------------------------------------------- Request
SamplingArgs RequestOptions::Resolve() const {
  SamplingArgs a;
  if (!do_sample || top_k == 1 || temperature == 0.f) return a;  // greedy
  a.temperature = temperature;
  const bool use_p = top_p > 0.f && top_p < 1.f;
  if (top_k > 1 && use_p) { a.top_k = top_k; a.top_p = top_p; }
  else if (top_k > 1) { a.top_k = top_k; a.top_p = 1.f; }
  else { a.top_k = -1; a.top_p = use_p ? top_p : 1.f; }
  return a;
}

Request::Request(uint64_t id, RequestOptions opt, std::vector<int32_t> eos)
    : id_(id), opt_(opt), eos_ids_(std::move(eos)) {
  if (opt_.batch_size != 1) throw std::runtime_error("Engine requests must use batch_size 1");
  if (opt_.num_beams != 1) throw std::runtime_error("Engine requests do not support beam search");
  if (opt_.random_seed >= 0) seed_ = uint64_t(opt_.random_seed);
  else { std::random_device rd; seed_ = (uint64_t(rd()) << 32) | rd(); }
}

void Request::AddTokens(const int32_t* ids, size_t n) {
  if (status_ != RequestStatus::kUnassigned)
    throw std::runtime_error("add_tokens: tokens can only be added before the request is given to an engine");
  if (n == 0) throw std::runtime_error("add_tokens: empty token list");
  tokens_.insert(tokens_.end(), ids, ids + n);
}

void Request::ContinueWith(const int32_t* ids, size_t n, int new_max_length) {
  if (status_ != RequestStatus::kTurnComplete)
    throw std::runtime_error("continue_with: the current turn is not complete");
  if (n == 0) throw std::runtime_error("continue_with: empty token list");
  if (new_max_length > 0) {
    // a new budget for the next turn (a turn that ended at max_length can only go on with a larger one)
    if (new_max_length < opt_.max_length) throw std::runtime_error("continue_with: max_length cannot shrink");
    opt_.max_length = new_max_length;
  }
  if (int(tokens_.size() + n) >= opt_.max_length)
    throw std::runtime_error("continue_with: max_length (cumulative across turns) would be exceeded");
  tokens_.insert(tokens_.end(), ids, ids + n);
  prefill_ = true;
  status_ = RequestStatus::kAssigned;
}

int Request::SetDraft(const int32_t* ids, size_t n) {
  if ((status_ != RequestStatus::kActive && status_ != RequestStatus::kAssigned) || prefill_ || draft_ != 0 || Pending() != 1) return 0;
  const int room = opt_.max_length - int(tokens_.size()) - 1;    // the token after the drafts needs a place too
  const int take = std::max(0, std::min(int(n), room));
  tokens_.insert(tokens_.end(), ids, ids + take);
  draft_ = take;
  return take;
}

int32_t Request::PopUnseen() {
  if (unseen_.empty()) throw std::runtime_error("get_unseen_token: no unseen tokens");
  int32_t t = unseen_.front();
  unseen_.pop_front();
  return t;
}

// ----------------------------------------------------------------------------------- EngineCore
EngineCore::EngineCore(EngineOptions opt) : opt_(std::move(opt)), pool_(opt_.num_blocks) {
  if (opt_.block_size <= 0 || opt_.num_blocks <= 0 || opt_.max_batch_size <= 0 || opt_.max_scheduled_tokens <= 0)
    throw std::invalid_argument("engine: block_size, num_blocks, max_batch_size and max_scheduled_tokens must be > 0");
  if (opt_.window_size > 0) {
    // Ring of R blocks per request: holds one step's chunk plus the window behind it.
    int chunk = opt_.max_scheduled_tokens;
    ring_blocks_ = (chunk + opt_.window_size - 1 + opt_.block_size - 1) / opt_.block_size;
    if (opt_.num_window_blocks <= 0) opt_.num_window_blocks = ring_blocks_ * opt_.max_batch_size;
    wpool_ = std::make_unique<BlockPool>(opt_.num_window_blocks);
  }
}

std::shared_ptr<Request> EngineCore::CreateRequest(RequestOptions o) {
  return std::make_shared<Request>(next_id_++, o, opt_.eos_ids);
}

void EngineCore::AddRequest(const std::shared_ptr<Request>& r) {
  if (!healthy_) throw std::runtime_error("engine is unhealthy after a fatal execution failure");
  if (r->status_ != RequestStatus::kUnassigned) throw std::runtime_error("add_request: request was already added to an engine");
  if (r->tokens_.empty()) throw std::runtime_error("add_request: request has no tokens");
  if (r->opt_.max_length <= 0) throw std::runtime_error("add_request: max_length must be > 0");
  if (int(r->tokens_.size()) >= r->opt_.max_length)
    throw std::runtime_error("add_request: prompt length " + std::to_string(r->tokens_.size()) +
                             " leaves no room under max_length " + std::to_string(r->opt_.max_length));
  if (opt_.static_batching && r->opt_.chunk_size > 0)
    throw std::runtime_error("search.chunk_size requires dynamic batching; the static batch scheduler cannot chunk a prefill.");
  r->status_ = RequestStatus::kAssigned;
  requests_.push_back(r);
  ++metrics_.requests_admitted;
}

void EngineCore::ReleaseRequestBlocks(Request& r) {
  for (int b : r.blocks_) pool_.Free(b);
  r.blocks_.clear();
  if (wpool_) for (int b : r.window_blocks_) wpool_->Free(b);
  r.window_blocks_.clear();
  r.resident_ = false;
}

void EngineCore::RemoveRequest(const std::shared_ptr<Request>& r) {
  if (open_)
    for (auto& e : plan_.entries)
      if (e.request == r) throw std::runtime_error("remove_request: request is part of the step in flight");
  auto it = std::find(requests_.begin(), requests_.end(), r);
  if (it == requests_.end()) return;
  ReleaseRequestBlocks(*r);
  r->status_ = RequestStatus::kClosed;
  requests_.erase(it);
  ready_.erase(std::remove(ready_.begin(), ready_.end(), r), ready_.end());
}

bool EngineCore::HasPendingRequests() const {
  if (!ready_.empty()) return true;
  for (auto& r : requests_)
    if (r->status_ == RequestStatus::kAssigned || r->status_ == RequestStatus::kActive || r->HasUnseen()) return true;
  return false;
}

const StepPlan& EngineCore::Plan() {
  if (!healthy_) throw std::runtime_error("engine is unhealthy after a fatal execution failure");
  if (open_) throw std::logic_error("Plan: previous step transaction is still open");
  plan_ = StepPlan{};
  reserved_.clear();

  // Candidates: residents first (admission order), then waiting requests; decodes before prefills.
  std::vector<std::shared_ptr<Request>> cands;
  auto executable = [](const Request& r) {
    return (r.status_ == RequestStatus::kAssigned || r.status_ == RequestStatus::kActive) && r.Pending() > 0;
  };
  for (auto& r : requests_) if (r->resident_ && executable(*r)) cands.push_back(r);
  if (opt_.static_batching) {
    // Static batching (reference: src/engine/scheduler.cpp:57-113): a batch runs to completion before the next one is
    // admitted; the next batch is the first 4 waiting requests, or 2, or 1, whichever the cache can hold at full length.
    if (cands.empty()) {
      std::vector<std::shared_ptr<Request>> waiting;
      for (auto& r : requests_) if (!r->resident_ && executable(*r)) waiting.push_back(r);
      constexpr size_t kStaticBatch = 4;
      for (size_t n = std::min({kStaticBatch, waiting.size(), size_t(opt_.max_batch_size)}); n != 0; n /= 2) {
        int blocks = 0;
        for (size_t i = 0; i < n; ++i)
          blocks += BlocksFor(std::max(waiting[i]->opt_.max_length, int(waiting[i]->tokens_.size())));
        if (blocks <= pool_.FreeCount() && (!wpool_ || int(n) * ring_blocks_ <= wpool_->FreeCount())) {
          cands.assign(waiting.begin(), waiting.begin() + long(n));
          break;
        }
      }
      if (cands.empty() && !waiting.empty()) {
        // not even one request fits at full length: a request larger than the whole pool can never run
        auto& r = waiting.front();
        if (BlocksFor(std::max(r->opt_.max_length, int(r->tokens_.size()))) > pool_.Total()) plan_.unserviceable.push_back(r);
        else ++plan_.deferred;
      }
    }
  } else {
    for (auto& r : requests_) if (!r->resident_ && executable(*r)) cands.push_back(r);
  }
  std::stable_partition(cands.begin(), cands.end(), [](const std::shared_ptr<Request>& r) { return !r->prefill_; });

  const int limit = std::min(opt_.max_scheduled_tokens, opt_.max_batch_size);
  for (auto& r : cands) {
    if (int(plan_.entries.size()) >= limit) break;
    // static batching owns the blocks of the whole max_length from the first step (the contiguous cache of the reference)
    const int need_total = BlocksFor(opt_.static_batching ? std::max(r->opt_.max_length, int(r->tokens_.size())) : int(r->tokens_.size()));
    if (need_total > pool_.Total() || (wpool_ && ring_blocks_ > wpool_->Total())) {
      plan_.unserviceable.push_back(r);
      continue;
    }
    Reserved res;
    int need = need_total - int(r->blocks_.size());
    bool reserved = false;
    if (opt_.lookahead > 0 && !r->prefill_) {
      // the block of the next positions too (never past max_length or the pool): kept by the request once committed
      const int ahead = std::min(int(r->tokens_.size()) + opt_.lookahead, std::max(r->opt_.max_length, int(r->tokens_.size())));
      const int want = std::min(BlocksFor(ahead), pool_.Total()) - int(r->blocks_.size());
      if (want > need) reserved = pool_.Reserve(want, res.blocks);
    }
    if (!reserved && need > 0 && !pool_.Reserve(need, res.blocks)) { ++plan_.deferred; continue; }
    if (wpool_) {
      const int wneed = ring_blocks_ - int(r->window_blocks_.size());
      if (wneed > 0 && !wpool_->Reserve(wneed, res.wblocks)) {
        for (int b : res.blocks) pool_.Release(b);
        ++plan_.deferred;
        continue;
      }
    }
    PlanEntry e;
    e.request = r;
    e.num_tokens = 1;
    e.processed_before = r->processed_;
    e.is_prefill = r->prefill_;
    e.newly_admitted = !r->resident_;
    plan_.entries.push_back(std::move(e));
    reserved_.push_back(std::move(res));
  }

  for (auto& r : plan_.unserviceable) {
    ReleaseRequestBlocks(*r);
    r->status_ = RequestStatus::kClosed;
    requests_.erase(std::remove(requests_.begin(), requests_.end(), r), requests_.end());
    ++metrics_.unserviceable;
  }

  if (plan_.entries.empty()) {
    if (!plan_.unserviceable.empty()) plan_.outcome = StepOutcome::kUnserviceableRequest;
    else if (plan_.deferred > 0) { plan_.outcome = StepOutcome::kCapacityDeferred; ++metrics_.steps_deferred; }
    else plan_.outcome = StepOutcome::kNoWork;
    return plan_;
  }

  // Token budget: one token each, then staged drafts, then prefills share what is left in plan order.
  int budget = opt_.max_scheduled_tokens - int(plan_.entries.size());
  for (auto& e : plan_.entries) {
    if (e.is_prefill || e.request->draft_ == 0) continue;
    if (e.request->draft_ > budget) {           // no room to verify the proposal this step: drop it
      e.request->tokens_.resize(e.request->tokens_.size() - size_t(e.request->draft_));
      e.request->draft_ = 0;
      continue;
    }
    e.num_tokens += e.request->draft_;
    budget -= e.request->draft_;
  }
  for (auto& e : plan_.entries) {
    if (!e.is_prefill) continue;
    int cap = e.request->Pending();
    if (e.request->opt_.chunk_size > 0) cap = std::min(cap, e.request->opt_.chunk_size);
    int extra = std::min(cap - 1, budget);
    e.num_tokens += extra;
    budget -= extra;
  }

  int off = 0;
  plan_.graph_eligible = true;
  plan_.lookahead_ok = opt_.lookahead > 0 && opt_.lookahead_execution && !wpool_;
  uint64_t sig = 1469598103934665603ull, nsig = 1469598103934665603ull;
  auto mix = [](uint64_t h, uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); return h * 1099511628211ull; };
  for (size_t i = 0; i < plan_.entries.size(); ++i) {
    const PlanEntry& e = plan_.entries[i];
    const Request& r = *e.request;
    sig = mix(mix(sig, r.id_), uint64_t(e.processed_before));
    nsig = mix(mix(nsig, r.id_), uint64_t(e.processed_before + 1));
    const int owned = int(r.blocks_.size() + reserved_[i].blocks.size());
    plan_.lookahead_ok = plan_.lookahead_ok && !e.is_prefill && e.num_tokens == 1 && int(r.tokens_.size()) + 1 < r.opt_.max_length &&
                         owned >= BlocksFor(int(r.tokens_.size()) + 1);
  }
  plan_.signature = sig;
  plan_.next_signature = nsig;
  for (auto& e : plan_.entries) {
    e.packed_offset = off;
    e.logits_row = off + e.num_tokens - 1;
    e.samples = (e.num_tokens == e.request->Pending());
    off += e.num_tokens;
    plan_.max_query_len = std::max(plan_.max_query_len, e.num_tokens);
    plan_.max_kv_len = std::max(plan_.max_kv_len, e.processed_before + e.num_tokens);
    plan_.graph_eligible &= (!e.is_prefill && e.num_tokens == 1);
    // checkpoint
    Request& r = *e.request;
    r.saved_ = Request::Saved{r.tokens_.size(), r.processed_, r.unseen_.size(), r.status_, r.prefill_,
                              r.blocks_.size(), r.window_blocks_.size()};
  }
  plan_.token_count = off;
  plan_.block_table_columns = BlocksFor(plan_.max_kv_len);
  plan_.outcome = StepOutcome::kPlanned;
  open_ = true;
  return plan_;
}

void EngineCore::Pack(const PackBuffers& buf) const {
  if (!open_) throw std::logic_error("Pack: no open step");
  const int B = int(plan_.entries.size());
  if (B > buf.max_batch || plan_.token_count > buf.max_tokens || plan_.block_table_columns > buf.table_columns)
    throw std::runtime_error("Pack: step exceeds the staging buffer capacity");
  const int bs = opt_.block_size, cols = buf.table_columns;
  buf.cu_seqlens[0] = 0;
  for (int i = 0; i < B; ++i) {
    const PlanEntry& e = plan_.entries[size_t(i)];
    const Request& r = *e.request;
    const Reserved& res = reserved_[size_t(i)];
    auto block_at = [&](int col) -> int {
      size_t held = r.blocks_.size();
      if (size_t(col) < held) return r.blocks_[size_t(col)];
      size_t k = size_t(col) - held;
      return k < res.blocks.size() ? res.blocks[k] : -1;
    };
    auto wblock_at = [&](int ring_idx) -> int {
      size_t held = r.window_blocks_.size();
      if (size_t(ring_idx) < held) return r.window_blocks_[size_t(ring_idx)];
      size_t k = size_t(ring_idx) - held;
      return k < res.wblocks.size() ? res.wblocks[k] : -1;
    };
    for (int t = 0; t < e.num_tokens; ++t) {
      const int pos = e.processed_before + t, idx = e.packed_offset + t;
      buf.input_ids[idx] = r.tokens_[size_t(pos)];
      buf.positions[idx] = pos;
      buf.token_row[idx] = i;
      buf.slot_mapping[idx] = block_at(pos / bs) * bs + pos % bs;
      if (buf.slot_mapping_w && wpool_) buf.slot_mapping_w[idx] = wblock_at((pos / bs) % ring_blocks_) * bs + pos % bs;
    }
    buf.cu_seqlens[i + 1] = e.packed_offset + e.num_tokens;
    buf.past_lens[i] = e.processed_before;
    buf.logits_rows[i] = e.logits_row;
    // with look-ahead the table also shows the block of the next positions (block_at gives -1 where none is owned)
    const int used_cols = std::min(cols, BlocksFor(e.processed_before + e.num_tokens + (e.is_prefill ? 0 : opt_.lookahead)));
    for (int c = 0; c < cols; ++c) buf.block_table[size_t(i) * cols + c] = c < used_cols ? block_at(c) : -1;
    if (buf.block_table_w && wpool_)
      for (int c = 0; c < cols; ++c) buf.block_table_w[size_t(i) * cols + c] = c < used_cols ? wblock_at(c % ring_blocks_) : -1;
    SamplingArgs a = r.opt_.Resolve();
    buf.top_k[i] = a.top_k;
    buf.top_p[i] = a.top_p;
    buf.temperature[i] = a.temperature;
    buf.seeds[i] = r.seed_;
    buf.sample_pos[i] = int(r.tokens_.size()) - r.draft_;      // position of the first token this step decides
  }
}

StepOutcome EngineCore::Commit(const int32_t* tokens, size_t n) {
  if (!open_) throw std::logic_error("Commit: no open step");
  if (n != plan_.entries.size()) throw std::invalid_argument("Commit: one token per planned entry is required");
  for (size_t i = 0; i < plan_.entries.size(); ++i) {
    PlanEntry& e = plan_.entries[i];
    Request& r = *e.request;
    Reserved& res = reserved_[i];
    for (int b : res.blocks) { pool_.Commit(b); r.blocks_.push_back(b); }
    if (wpool_) for (int b : res.wblocks) { wpool_->Commit(b); r.window_blocks_.push_back(b); }
    r.resident_ = true;
    r.processed_ += e.num_tokens;
    r.status_ = RequestStatus::kActive;
    r.saved_.reset();
    metrics_.tokens_scheduled += uint64_t(e.num_tokens);
    if (!e.samples) continue;
    r.prefill_ = false;
    const int32_t tok = tokens[i];
    // A sampled end-of-sequence token is part of the sequence and of the stream the caller reads, as in the reference
    // engine (src/engine/request.cpp CommitStep pushes whatever the search appended, and GreedySearch_Cpu appends the
    // EOS it selected, src/search.cpp:266-296): it ends the turn, is never fed to the sampler again, and is the first
    // token of the prefill of a continued turn.
    const bool eos = std::find(r.eos_ids_.begin(), r.eos_ids_.end(), tok) != r.eos_ids_.end();
    bool complete = eos;
    if (int(r.tokens_.size()) < r.opt_.max_length) {
      r.tokens_.push_back(tok);
      r.unseen_.push_back(tok);
      ++metrics_.tokens_generated;
    }
    if (int(r.tokens_.size()) >= r.opt_.max_length) complete = true;
    if (complete) { r.status_ = RequestStatus::kTurnComplete; ++metrics_.requests_completed; }
    if (std::find(ready_.begin(), ready_.end(), e.request) == ready_.end()) ready_.push_back(e.request);
  }
  open_ = false;
  ++metrics_.steps_committed;
  plan_.outcome = StepOutcome::kCommitted;
  return plan_.outcome;
}

StepOutcome EngineCore::CommitSpeculative(const int32_t* accepted, const int32_t* tokens, size_t n) {
  if (!open_) throw std::logic_error("CommitSpeculative: no open step");
  if (n != plan_.entries.size()) throw std::invalid_argument("CommitSpeculative: one entry per planned entry is required");
  for (size_t i = 0; i < n; ++i) {
    Request& r = *plan_.entries[i].request;
    const int staged = plan_.entries[i].num_tokens > 1 && !plan_.entries[i].is_prefill ? r.draft_ : 0;
    if (accepted[i] < 0 || accepted[i] > staged) throw std::invalid_argument("CommitSpeculative: accepted count out of range");
  }
  // Rejected drafts leave the sequence and the number of fed tokens shrinks to what the cache keeps; then every entry is an
  // ordinary entry that sampled tokens[i], except that the accepted drafts are generated output too.
  std::vector<char> ended_on_draft(n, 0);
  for (size_t i = 0; i < n; ++i) {
    PlanEntry& e = plan_.entries[i];
    Request& r = *e.request;
    if (e.is_prefill || r.draft_ == 0 || e.num_tokens == 1) continue;
    const int staged = r.draft_, keep = accepted[i];
    const size_t base = r.tokens_.size() - size_t(staged);       // tokens before the drafts (the last one was pending)
    int surfaced = 0;
    bool ended = false;
    for (int j = 0; j < keep && !ended; ++j) {                   // accepted drafts are output; one that ends the sequence stops it
      const int32_t t = r.tokens_[base + size_t(j)];
      r.unseen_.push_back(t);
      ++metrics_.tokens_generated;
      ++surfaced;
      ended = std::find(r.eos_ids_.begin(), r.eos_ids_.end(), t) != r.eos_ids_.end();
    }
    r.tokens_.resize(base + size_t(surfaced));
    r.draft_ = 0;
    e.num_tokens = 1 + surfaced;                                  // slots the cache keeps: the pending token and the kept drafts
    if (ended) {
      // the turn ends on an accepted draft: nothing is sampled after it; the token itself is fed when the turn continues
      e.num_tokens = surfaced;
      e.samples = false;
      ended_on_draft[i] = 1;
    }
  }
  // the ordinary commit appends tokens[i] where the entry samples; entries that ended on a draft complete their turn here
  const StepOutcome out = Commit(tokens, n);
  for (size_t i = 0; i < n; ++i) {
    if (!ended_on_draft[i]) continue;
    Request& r = *plan_.entries[i].request;
    if (r.status_ != RequestStatus::kTurnComplete) {
      r.status_ = RequestStatus::kTurnComplete;
      ++metrics_.requests_completed;
      if (std::find(ready_.begin(), ready_.end(), plan_.entries[i].request) == ready_.end()) ready_.push_back(plan_.entries[i].request);
    }
  }
  return out;
}

StepOutcome EngineCore::Abort(FailureKind kind, const std::string&) {
  if (!open_) throw std::logic_error("Abort: no open step");
  for (size_t i = 0; i < plan_.entries.size(); ++i) {
    Request& r = *plan_.entries[i].request;
    for (int b : reserved_[i].blocks) pool_.Release(b);
    if (wpool_) for (int b : reserved_[i].wblocks) wpool_->Release(b);
    if (r.saved_) {
      r.tokens_.resize(r.saved_->token_count);
      r.processed_ = r.saved_->processed;
      while (r.unseen_.size() > r.saved_->unseen) r.unseen_.pop_back();
      r.status_ = r.saved_->status;
      r.prefill_ = r.saved_->prefill;
      r.saved_.reset();
    }
  }
  reserved_.clear();
  open_ = false;
  ++metrics_.steps_aborted;
  switch (kind) {
    case FailureKind::kRetryableBeforeExecution:
    case FailureKind::kRetryableDuringExecution: plan_.outcome = StepOutcome::kRetryableBatchAbort; break;
    case FailureKind::kCapacityExceeded: plan_.outcome = StepOutcome::kExecutionCapacityExceeded; break;
    case FailureKind::kPostProcessing: plan_.outcome = StepOutcome::kExecutionContractFailure; break;
    case FailureKind::kFatal: plan_.outcome = StepOutcome::kFatalExecutionFailure; healthy_ = false; break;
  }
  return plan_.outcome;
}

std::shared_ptr<Request> EngineCore::NextReady() {
  while (!ready_.empty()) {
    auto r = ready_.front();
    ready_.pop_front();
    if (r->status_ == RequestStatus::kClosed) continue;
    return r;
  }
  return nullptr;
}

void EngineCore::CheckInvariants() const {
  auto check_pool = [&](const BlockPool& pool, bool windowed) {
    std::vector<int> owners(size_t(pool.Total()), 0);
    for (auto& r : requests_)
      for (int b : (windowed ? r->window_blocks_ : r->blocks_)) {
        if (b < 0 || b >= pool.Total()) throw std::logic_error("invariant: request holds an out-of-range block id");
        if (pool.StateOf(b) != BlockPool::State::kCommitted) throw std::logic_error("invariant: request block is not committed in the pool");
        if (++owners[size_t(b)] > 1) throw std::logic_error("invariant: block owned by two requests");
      }
    int reserved_listed = 0;
    if (open_)
      for (auto& res : reserved_)
        for (int b : (windowed ? res.wblocks : res.blocks)) {
          if (pool.StateOf(b) != BlockPool::State::kReserved) throw std::logic_error("invariant: reservation lists a block that is not reserved");
          if (owners[size_t(b)]) throw std::logic_error("invariant: block both reserved and committed");
          ++reserved_listed;
        }
    int free_n = 0, res_n = 0, com_n = 0;
    for (int b = 0; b < pool.Total(); ++b) {
      switch (pool.StateOf(b)) {
        case BlockPool::State::kFree: ++free_n; break;
        case BlockPool::State::kReserved: ++res_n; break;
        case BlockPool::State::kCommitted: ++com_n; if (!owners[size_t(b)]) throw std::logic_error("invariant: committed block has no owner (leak)"); break;
      }
    }
    if (free_n != pool.FreeCount()) throw std::logic_error("invariant: free list size disagrees with block states");
    if (res_n != reserved_listed) throw std::logic_error("invariant: reserved blocks outside an open transaction");
  };
  check_pool(pool_, false);
  if (wpool_) check_pool(*wpool_, true);
  for (auto& r : requests_) {
    if (r->processed_ < 0 || r->processed_ > int(r->tokens_.size())) throw std::logic_error("invariant: processed length out of range");
    if (r->resident_ && BlocksFor(r->processed_) > int(r->blocks_.size())) throw std::logic_error("invariant: committed KV slots exceed owned blocks");
    if ((r->status_ == RequestStatus::kAssigned || r->status_ == RequestStatus::kActive) && r->Pending() <= 0)
      throw std::logic_error("invariant: executable request has no pending token");
  }
}

}  // namespace ogb::engine
