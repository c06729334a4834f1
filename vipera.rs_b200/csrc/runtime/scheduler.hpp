// Continuous batching: which requests run in the next step and with which tokens.
//
// The reference's engine admits turns oldest-first up to a batch cap, runs prompt chunks
// and single decode tokens in alternating steps, samples in request order with one
// generator per request, finishes on an end token, on the token limit or on a full cache,
// and fails the requests of a step whose reservation cannot be met
// (crates/vipera-runtime/src/engine.rs:396-424, 606-765, 1063-1140).  This scheduler keeps
// the admission, finishing and per-request generators.  It differs in three decisions:
//   * portions of prompts and decode tokens share one step, under a budget of tokens;
//   * a portion may be any length from one token up, cut where the budget or the free
//     pages end;
//   * when pages run out, the request admitted last is put back at the head of the
//     waiting line with its pages freed, to be computed again later; only a request that
//     is alone and still cannot grow ends, with reason "length".
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <string>
#include <vector>

#include "cache_manager.hpp"
#include "sampler.hpp"

namespace vipera {

struct RequestParams {
  SamplerConfig sampler;
  int max_new_tokens = 32;
  std::vector<int32_t> eos_ids;
  int recent_window = 128;  // tokens the penalties look back over (engine.rs:37)
};

struct SchedulerConfig {
  int max_num_seqs = 4;          // requests running at once (engine.rs:1125-1140)
  int max_tokens_per_step = 512; // budget of one step
  int max_portion = 512;         // longest portion of one prompt in one step
  int max_model_len = 0;         // 0: bounded by the cache only
  bool reuse_prefixes = true;    // share the pages of prompt prefixes seen before (where the cache can)
};

struct StepEntry {
  int64_t request = 0;
  int start = 0;   // position of the entry's first token
  int count = 0;   // tokens of this request in the step
  int state_slot = 0;
  bool fresh = false;  // first portion since (re)admission: per-request state starts anew
  bool wants_logits = false;
};

struct SampleRow {
  int64_t request = 0;
  int token_index = 0;  // index into StepPlan::tokens whose logits are sampled
  float temperature = 0, top_p = 1, min_p = 0;
  int top_k = 0;
  double uniform = 0;   // the request's next draw, taken only when temperature > 0
  // Ids whose logits the penalties change, with counts; empty when no penalty is set.
  std::vector<int32_t> penalty_ids;
  std::vector<int32_t> penalty_counts;
  float repetition_penalty = 1, presence_penalty = 0, frequency_penalty = 0;
  std::vector<std::pair<uint32_t, float>> logit_bias;
};

struct StepPlan {
  std::vector<StepEntry> entries;
  std::vector<int32_t> tokens;     // flat, entry after entry
  std::vector<int32_t> positions;  // same length
  std::vector<SampleRow> rows;     // in entry order
  std::vector<int64_t> preempted;  // put back to waiting while this plan was made
  bool empty() const { return entries.empty(); }
};

struct Finished {
  int64_t request = 0;
  std::string reason;  // "stop" | "length" | "cancelled" | "error"
  std::vector<int32_t> tokens;  // generated tokens, the end token included
  int prompt_tokens = 0;
  int processed_tokens = 0;  // tokens run through the model, recomputation included
  int reused_tokens = 0;     // prompt tokens taken from pages an earlier request computed
  int preemptions = 0;
};

struct StepOutcome {
  std::vector<std::pair<int64_t, int32_t>> tokens;  // (request, new token) in row order
  std::vector<Finished> finished;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, SchedulerConfig config);

  // Admission (engine.rs:396-424): a prompt must be non-empty, max_new_tokens at least
  // one, and prompt pages must fit the pool; else Infeasible / InvalidArgument.
  void add(int64_t request, std::vector<int32_t> prompt, RequestParams params);
  void cancel(int64_t request);  // pages are freed at once; reported by the next complete()
  bool has_work() const { return !waiting_.empty() || !running_.empty() || !cancelled_.empty(); }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }

  StepPlan schedule();
  // Whether the step after `plan` (made by schedule() and not yet completed) is known already:
  // every running request decodes greedily in `plan`, nobody waits, and none of them can end
  // with this step's token except by drawing an end token, and no row has penalties (they
  // depend on the token).  If so, the pages for the token after are reserved now and the caller may launch that step (the same requests, positions
  // one further, the tokens `plan` draws) before it has read `plan`'s tokens.  The scheduler's
  // own state does not change: complete() and the next schedule() go on as ever, and the
  // caller compares what schedule() then returns with what it launched.
  // `max_top_k`: rows that draw with a temperature are foreseen only with a top-k between 1 and
  // this bound (what the caller's sampler draws on the device without a second look at the
  // logits, which the step launched ahead overwrites); 0 foresees greedy rows only.
  bool plan_ahead(const StepPlan& plan, int max_top_k = 0);
  // The uniform draws that schedule() will hand the rows of the step after `plan` (one per row of
  // `plan`, 0 for greedy rows), looked at without being taken.
  std::vector<double> peek_uniforms(const StepPlan& plan) const;
  // `sampled[i]` is the token drawn for plan.rows[i].
  StepOutcome complete(const StepPlan& plan, const std::vector<int32_t>& sampled);
  // The step failed as a whole: its requests end with reason "error" and free their pages
  // (engine.rs:731-741).
  StepOutcome fail(const StepPlan& plan);

 private:
  struct Request {
    int64_t id = 0;
    std::vector<int32_t> tokens;  // prompt, then generated
    int prompt_len = 0;
    int processed = 0;
    int reused = 0;
    int preemptions = 0;
    uint64_t order = 0;  // admission order, for the choice of whom to put back
    bool fresh = true;
    RequestParams params;
    Rng rng;
  };

  bool preempt_latest(int64_t keep, StepPlan* plan);
  Finished finish(Request& request, const std::string& reason);
  void fill_row(Request& request, int token_index, SampleRow* row);

  CacheManager* cache_;
  SchedulerConfig config_;
  std::deque<Request> waiting_;
  std::map<int64_t, Request> running_;  // by id, so that entries and draws come in id order
  std::vector<Finished> cancelled_;
  uint64_t next_order_ = 0;
};

}  // namespace vipera
