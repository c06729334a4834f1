#include "scheduler.hpp"

#include <algorithm>

namespace vipera {

Scheduler::Scheduler(CacheManager* cache, SchedulerConfig config) : cache_(cache), config_(config) {
  if (cache == nullptr) throw InvalidArgument("a scheduler needs a cache manager");
  if (config_.max_num_seqs <= 0) throw InvalidArgument("max_num_seqs must be at least 1");
  if (config_.max_tokens_per_step <= 0) throw InvalidArgument("max_tokens_per_step must be at least 1");
  if (config_.max_portion <= 0) throw InvalidArgument("max_portion must be at least 1");
}

void Scheduler::add(int64_t request, std::vector<int32_t> prompt, RequestParams params) {
  if (prompt.empty()) throw InvalidArgument("a prompt needs at least one token");
  if (params.max_new_tokens < 1) throw InvalidArgument("max_new_tokens must be at least 1");
  try {
    params.sampler.validate();
  } catch (const std::invalid_argument& error) {
    throw InvalidArgument(error.what());
  }
  if (running_.count(request)) throw InvalidArgument("request id is already in use");
  for (const Request& other : waiting_)
    if (other.id == request) throw InvalidArgument("request id is already in use");
  int length = static_cast<int>(prompt.size());
  if (config_.max_model_len > 0 && length >= config_.max_model_len)
    throw Infeasible("prompt of " + std::to_string(length) + " tokens leaves no room under the limit of " +
                     std::to_string(config_.max_model_len) + " positions");
  if (!cache_->could_ever_fit(length + 1))
    throw Infeasible("prompt of " + std::to_string(length) + " tokens does not fit the cache of " +
                     std::to_string(cache_->capacity_tokens()) + " tokens");
  Request entry;
  entry.id = request;
  entry.prompt_len = length;
  entry.tokens = std::move(prompt);
  entry.rng = Rng(params.sampler.seed);
  entry.params = std::move(params);
  waiting_.push_back(std::move(entry));
}

void Scheduler::cancel(int64_t request) {
  auto it = running_.find(request);
  if (it != running_.end()) {
    cancelled_.push_back(finish(it->second, "cancelled"));
    running_.erase(it);
    return;
  }
  for (auto w = waiting_.begin(); w != waiting_.end(); ++w) {
    if (w->id != request) continue;
    cancelled_.push_back(finish(*w, "cancelled"));
    waiting_.erase(w);
    return;
  }
}

Finished Scheduler::finish(Request& request, const std::string& reason) {
  if (cache_->is_open(request.id)) cache_->close(request.id);
  Finished out;
  out.request = request.id;
  out.reason = reason;
  out.tokens.assign(request.tokens.begin() + request.prompt_len, request.tokens.end());
  out.prompt_tokens = request.prompt_len;
  out.processed_tokens = request.processed;
  out.reused_tokens = request.reused;
  out.preemptions = request.preemptions;
  return out;
}

bool Scheduler::preempt_latest(int64_t keep, StepPlan* plan) {
  auto victim = running_.end();
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if (it->first == keep) continue;
    if (victim == running_.end() || it->second.order > victim->second.order) victim = it;
  }
  if (victim == running_.end()) return false;
  Request request = std::move(victim->second);
  running_.erase(victim);
  cache_->close(request.id);
  for (auto e = plan->entries.begin(); e != plan->entries.end(); ++e) {
    if (e->request != request.id) continue;
    plan->entries.erase(e);
    break;
  }
  request.preemptions += 1;
  request.fresh = true;
  plan->preempted.push_back(request.id);
  waiting_.push_front(std::move(request));
  return true;
}

void Scheduler::fill_row(Request& request, int token_index, SampleRow* row) {
  const SamplerConfig& sampler = request.params.sampler;
  row->request = request.id;
  row->token_index = token_index;
  row->temperature = sampler.temperature;
  row->top_k = sampler.top_k;
  row->top_p = sampler.top_p;
  row->min_p = sampler.min_p;
  row->uniform = sampler.temperature > 0.0f ? request.rng.next_f64() : 0.0;
  if (!sampler.has_penalty()) return;
  int total = static_cast<int>(request.tokens.size());
  int recent = std::min(total, std::max(0, request.params.recent_window));
  Penalty penalty(sampler, request.tokens.data() + (total - recent), recent);
  for (const auto& item : penalty.counts()) {
    row->penalty_ids.push_back(static_cast<int32_t>(item.first));
    row->penalty_counts.push_back(static_cast<int32_t>(item.second));
  }
  row->repetition_penalty = sampler.repetition_penalty;
  row->presence_penalty = sampler.presence_penalty;
  row->frequency_penalty = sampler.frequency_penalty;
  row->logit_bias = penalty.bias();
}

StepPlan Scheduler::schedule() {
  StepPlan plan;
  // Entries are gathered per request first; the flat token arrays are built at the end,
  // because a request may be put back to waiting after its entry was made.
  for (size_t attempt = 0; attempt <= running_.size() + 1; ++attempt) {
    int used = 0;
    for (const StepEntry& entry : plan.entries) used += entry.count;
    std::vector<int64_t> ids;
    for (const auto& item : running_) ids.push_back(item.first);
    for (int64_t id : ids) {
      auto it = running_.find(id);
      if (it == running_.end()) continue;  // put back while an earlier request was served
      bool planned = false;
      for (const StepEntry& entry : plan.entries) planned = planned || entry.request == id;
      if (planned) continue;
      Request& request = it->second;
      int computed = cache_->computed(id);
      int remaining = static_cast<int>(request.tokens.size()) - computed;
      int budget = config_.max_tokens_per_step - used;
      int want = std::min({remaining, config_.max_portion, budget});
      if (want <= 0) continue;
      int target = computed + want;
      if (!cache_->fits(id, target)) {
        if (remaining == 1) {
          // A decode token needs a page: requests admitted later make room.
          while (!cache_->fits(id, target) && preempt_latest(id, &plan)) {
          }
          used = 0;
          for (const StepEntry& entry : plan.entries) used += entry.count;
          if (!cache_->fits(id, target)) {
            // Alone and still no page: the cache is this request's limit.
            cancelled_.push_back(finish(request, "length"));
            running_.erase(id);
            continue;
          }
        } else {
          target = cache_->longest_fit(id, target);
          want = target - computed;
          if (want <= 0) continue;  // waits for pages
        }
      }
      cache_->reserve(id, target);
      StepEntry entry;
      entry.request = id;
      entry.start = computed;
      entry.count = want;
      entry.state_slot = cache_->state_slot(id);
      entry.fresh = request.fresh;
      entry.wants_logits = target == static_cast<int>(request.tokens.size());
      plan.entries.push_back(entry);
      used += want;
    }
    if (!plan.entries.empty() || running_.empty()) break;
    // Every running request waits for pages that only another running request can give
    // back: the one admitted last starts over.  One request alone that cannot take a
    // single token more ends.
    if (!preempt_latest(-1, &plan)) break;
    if (running_.empty()) {
      // The one put back was alone; it cannot run, so it ends here.
      Request request = std::move(waiting_.front());
      waiting_.pop_front();
      plan.preempted.pop_back();
      cancelled_.push_back(finish(request, "length"));
      break;
    }
  }

  // Admission, oldest first, only in a step that put nobody back.
  int used = 0;
  for (const StepEntry& entry : plan.entries) used += entry.count;
  while (plan.preempted.empty() && !waiting_.empty() &&
         static_cast<int>(running_.size()) < config_.max_num_seqs &&
         used < config_.max_tokens_per_step && cache_->free_state_slots() > 0) {
    Request& head = waiting_.front();
    int length = static_cast<int>(head.tokens.size());
    cache_->open(head.id);
    // Pages of a prompt prefix an earlier request computed are shared, not computed again
    // (the reference copies them: engine.rs:432-491).
    const bool reuse = config_.reuse_prefixes && cache_->reuse();
    const int reused = reuse ? cache_->match(head.id, head.tokens.data(), length) : 0;
    const bool room = reuse ? cache_->fits(head.id, length) : cache_->admits(length, config_.max_portion);
    if (!room) {
      cache_->close(head.id);
      if (running_.empty()) {
        // Nothing runs and it still does not fit: it never will.
        Request request = std::move(waiting_.front());
        waiting_.pop_front();
        cancelled_.push_back(finish(request, "length"));
        continue;
      }
      break;
    }
    int want = std::min({length - reused, config_.max_portion, config_.max_tokens_per_step - used});
    want = cache_->longest_fit(head.id, reused + want) - reused;
    if (want <= 0) {
      cache_->close(head.id);
      break;
    }
    cache_->reserve(head.id, reused + want);
    Request request = std::move(waiting_.front());
    waiting_.pop_front();
    request.order = next_order_++;
    request.reused += reused;
    StepEntry entry;
    entry.request = request.id;
    entry.start = reused;
    entry.count = want;
    entry.state_slot = cache_->state_slot(request.id);
    entry.fresh = true;
    entry.wants_logits = reused + want == length;
    plan.entries.push_back(entry);
    used += want;
    running_.emplace(request.id, std::move(request));
  }

  std::sort(plan.entries.begin(), plan.entries.end(),
            [](const StepEntry& a, const StepEntry& b) { return a.request < b.request; });
  for (const StepEntry& entry : plan.entries) {
    Request& request = running_.at(entry.request);
    for (int i = 0; i < entry.count; ++i) {
      plan.tokens.push_back(request.tokens[entry.start + i]);
      plan.positions.push_back(entry.start + i);
    }
    if (entry.wants_logits) {
      SampleRow row;
      fill_row(request, static_cast<int>(plan.tokens.size()) - 1, &row);
      plan.rows.push_back(std::move(row));
    }
  }
  return plan;
}

std::vector<double> Scheduler::peek_uniforms(const StepPlan& plan) const {
  std::vector<double> draws;
  draws.reserve(plan.rows.size());
  for (const SampleRow& row : plan.rows) {
    auto it = running_.find(row.request);
    if (it == running_.end() || it->second.params.sampler.temperature <= 0.0f) {
      draws.push_back(0.0);
      continue;
    }
    Rng generator = it->second.rng;  // a copy: the request's own generator is not advanced
    draws.push_back(generator.next_f64());
  }
  return draws;
}

bool Scheduler::plan_ahead(const StepPlan& plan, int max_top_k) {
  if (plan.entries.empty() || !plan.preempted.empty() || !waiting_.empty() || !cancelled_.empty()) return false;
  if (plan.entries.size() != running_.size() || plan.rows.size() != plan.entries.size()) return false;
  for (const StepEntry& entry : plan.entries) {
    auto it = running_.find(entry.request);
    if (it == running_.end()) return false;
    const Request& request = it->second;
    const int length = static_cast<int>(request.tokens.size());  // before this step's token
    if (entry.count != 1 || !entry.wants_logits || entry.start + 1 != length) return false;
    const SamplerConfig& sampler = request.params.sampler;
    if (sampler.has_penalty()) return false;
    if (sampler.temperature > 0.0f && (sampler.top_k < 1 || sampler.top_k > max_top_k)) return false;
    // the ends complete() finds without looking at the token
    if (length + 1 - request.prompt_len >= request.params.max_new_tokens) return false;
    if (config_.max_model_len > 0 && length + 1 >= config_.max_model_len) return false;
    if (!cache_->could_ever_fit(length + 1)) return false;
  }
  for (const StepEntry& entry : plan.entries) {
    if (!cache_->fits(entry.request, entry.start + 2)) return false;  // what was reserved so far stays: harmless
    cache_->reserve(entry.request, entry.start + 2);
  }
  return true;
}

StepOutcome Scheduler::complete(const StepPlan& plan, const std::vector<int32_t>& sampled) {
  if (sampled.size() != plan.rows.size())
    throw InvalidArgument("complete() needs one sampled token for each row of the plan");
  StepOutcome outcome;
  outcome.finished = std::move(cancelled_);
  cancelled_.clear();
  for (const StepEntry& entry : plan.entries) {
    auto it = running_.find(entry.request);
    if (it == running_.end()) continue;  // cancelled while the step ran
    cache_->commit(entry.request, entry.start + entry.count);
    it->second.processed += entry.count;
    it->second.fresh = false;
    // full pages of the prompt become available to requests that begin the same way
    if (config_.reuse_prefixes && cache_->reuse())
      cache_->publish(entry.request, it->second.tokens.data(),
                      std::min(entry.start + entry.count, it->second.prompt_len));
  }
  for (size_t i = 0; i < plan.rows.size(); ++i) {
    auto it = running_.find(plan.rows[i].request);
    if (it == running_.end()) continue;
    Request& request = it->second;
    int32_t token = sampled[i];
    request.tokens.push_back(token);
    outcome.tokens.push_back({request.id, token});
    int generated = static_cast<int>(request.tokens.size()) - request.prompt_len;
    int length = static_cast<int>(request.tokens.size());
    const std::vector<int32_t>& eos = request.params.eos_ids;
    std::string reason;
    if (std::find(eos.begin(), eos.end(), token) != eos.end()) reason = "stop";
    else if (generated >= request.params.max_new_tokens) reason = "length";
    else if (config_.max_model_len > 0 && length >= config_.max_model_len) reason = "length";
    else if (!cache_->could_ever_fit(length)) reason = "length";
    if (!reason.empty()) {
      outcome.finished.push_back(finish(request, reason));
      running_.erase(it);
    }
  }
  return outcome;
}

StepOutcome Scheduler::fail(const StepPlan& plan) {
  StepOutcome outcome;
  outcome.finished = std::move(cancelled_);
  cancelled_.clear();
  for (const StepEntry& entry : plan.entries) {
    auto it = running_.find(entry.request);
    if (it == running_.end()) continue;
    outcome.finished.push_back(finish(it->second, "error"));
    running_.erase(it);
  }
  return outcome;
}

}  // namespace vipera
