#include "sampler.hpp"

#include <algorithm>
#include <cmath>
#include <queue>

namespace vipera {

namespace {
uint64_t splitmix64(uint64_t state) {
  state += 0x9E3779B97F4A7C15ull;
  uint64_t z = state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct Candidate {
  uint32_t id;
  float value;
};

// Best first: higher value, then lower id (crates/vipera-sampler/src/lib.rs:440-444).
bool better(const Candidate& a, const Candidate& b) {
  if (a.value != b.value) return a.value > b.value;
  return a.id < b.id;
}

// The `bound` best finite penalised logits, best first; bound 0 sorts all of them
// (crates/vipera-sampler/src/lib.rs:484-527).
std::vector<Candidate> top_candidates(const float* logits, int vocab, const Penalty& penalty,
                                      int bound) {
  std::vector<Candidate> out;
  if (bound == 0 || bound >= vocab) {
    out.reserve(vocab);
    for (int id = 0; id < vocab; ++id) {
      if (!std::isfinite(logits[id])) continue;
      float value = penalty.apply(id, logits[id]);
      if (std::isfinite(value)) out.push_back({static_cast<uint32_t>(id), value});
    }
    std::sort(out.begin(), out.end(), better);
    return out;
  }
  // A heap whose top is the worst kept candidate.
  auto worse_on_top = [](const Candidate& a, const Candidate& b) { return better(a, b); };
  std::priority_queue<Candidate, std::vector<Candidate>, decltype(worse_on_top)> heap(worse_on_top);
  for (int id = 0; id < vocab; ++id) {
    if (!std::isfinite(logits[id])) continue;
    float value = penalty.apply(id, logits[id]);
    if (!std::isfinite(value)) continue;
    Candidate candidate{static_cast<uint32_t>(id), value};
    if (static_cast<int>(heap.size()) < bound) {
      heap.push(candidate);
    } else if (better(candidate, heap.top())) {
      heap.pop();
      heap.push(candidate);
    }
  }
  out.resize(heap.size());
  for (size_t i = heap.size(); i-- > 0;) {
    out[i] = heap.top();
    heap.pop();
  }
  return out;
}

// Length of the shortest head whose weights reach `target`, or -1
// (crates/vipera-sampler/src/lib.rs:421-430).
int mass_cut(const std::vector<Candidate>& weights, float target) {
  float cumulative = 0.0f;
  for (size_t i = 0; i < weights.size(); ++i) {
    cumulative += weights[i].value;
    if (cumulative >= target) return static_cast<int>(i) + 1;
  }
  return -1;
}
}  // namespace

void Rng::reseed(uint64_t seed) { state_ = splitmix64(seed ^ 0x9E3779B97F4A7C15ull); }

uint64_t Rng::next_u64() {
  uint64_t x = state_;
  x ^= x >> 12;
  x ^= x << 25;
  x ^= x >> 27;
  state_ = x;
  return x * 0x2545F4914F6CDD1Dull;
}

double Rng::next_f64() {
  return static_cast<double>(next_u64() >> 11) / static_cast<double>(1ull << 53);
}

void SamplerConfig::validate() const {
  if (!std::isfinite(temperature) || temperature < 0.0f)
    throw std::invalid_argument("temperature must be a finite number at or above 0");
  if (top_k < 0) throw std::invalid_argument("top_k must be at least 0");
  if (!std::isfinite(top_p) || top_p <= 0.0f || top_p > 1.0f)
    throw std::invalid_argument("top_p must be greater than 0 and at most 1");
  if (!std::isfinite(min_p) || min_p < 0.0f || min_p >= 1.0f)
    throw std::invalid_argument("min_p must be at least 0 and below 1");
  if (!std::isfinite(repetition_penalty) || repetition_penalty <= 0.0f)
    throw std::invalid_argument("repetition_penalty must be a finite number above 0");
  if (!std::isfinite(presence_penalty) || presence_penalty < -2.0f || presence_penalty > 2.0f)
    throw std::invalid_argument("presence_penalty must be a finite number from -2 to 2");
  if (!std::isfinite(frequency_penalty) || frequency_penalty < -2.0f || frequency_penalty > 2.0f)
    throw std::invalid_argument("frequency_penalty must be a finite number from -2 to 2");
  if (logit_bias.size() > 16) throw std::invalid_argument("logit_bias takes at most 16 entries");
  for (const auto& bias : logit_bias)
    if (!std::isfinite(bias.second) || bias.second < -100.0f || bias.second > 100.0f)
      throw std::invalid_argument("logit_bias values must be finite numbers from -100 to 100");
}

Penalty::Penalty(const SamplerConfig& config, const int32_t* recent, int recent_count)
    : factor_(config.repetition_penalty),
      presence_(config.presence_penalty),
      frequency_(config.frequency_penalty) {
  bool counting = factor_ != 1.0f || presence_ != 0.0f || frequency_ != 0.0f;
  if (counting && recent_count > 0) {
    std::vector<uint32_t> ids(recent, recent + recent_count);
    std::sort(ids.begin(), ids.end());
    for (uint32_t id : ids) {
      if (!counts_.empty() && counts_.back().first == id) ++counts_.back().second;
      else counts_.push_back({id, 1u});
    }
  }
  bias_ = config.logit_bias;
  std::sort(bias_.begin(), bias_.end());
}

float Penalty::apply(uint32_t id, float logit) const {
  float value = logit;
  if (!counts_.empty()) {
    auto it = std::lower_bound(counts_.begin(), counts_.end(), std::make_pair(id, 0u));
    if (it != counts_.end() && it->first == id) {
      if (factor_ != 1.0f) value = value > 0.0f ? value / factor_ : value * factor_;
      value -= presence_ + frequency_ * static_cast<float>(it->second);
    }
  }
  if (!bias_.empty()) {
    auto it = std::lower_bound(bias_.begin(), bias_.end(), id,
                               [](const std::pair<uint32_t, float>& a, uint32_t b) { return a.first < b; });
    if (it != bias_.end() && it->first == id) value += it->second;
  }
  return value;
}

uint32_t draw_greedy(const float* logits, int vocab, const Penalty& penalty) {
  bool found = false;
  Candidate best{0, 0.0f};
  for (int id = 0; id < vocab; ++id) {
    if (!std::isfinite(logits[id])) continue;
    float value = penalty.apply(id, logits[id]);
    if (!std::isfinite(value)) continue;
    if (!found || value > best.value) {  // ids ascend, so a tie keeps the lower id
      best = {static_cast<uint32_t>(id), value};
      found = true;
    }
  }
  if (!found) throw SampleError("no finite logits to sample from");
  return best.id;
}

uint32_t draw_temperature(const float* logits, int vocab, const Penalty& penalty, float temperature,
                          int top_k, float top_p, float min_p, double uniform) {
  const float scale = 1.0f / temperature;
  const bool uncut = top_k == 0;
  std::vector<Candidate> weights = top_candidates(logits, vocab, penalty, uncut ? kNoCutCandidates : top_k);
  if (weights.empty()) throw SampleError("no finite logits to sample from");
  const float peak = weights[0].value * scale;
  float total = 0.0f;
  for (int id = 0; id < vocab; ++id) {
    if (!std::isfinite(logits[id])) continue;
    float value = penalty.apply(id, logits[id]);
    if (std::isfinite(value)) total += std::exp(value * scale - peak);
  }
  if (!(total > 0.0f) || !std::isfinite(total)) throw SampleError("the distribution has no mass");
  for (Candidate& c : weights) c.value = std::exp(c.value * scale - peak);
  const float target_mass = top_p * total;
  int cut = mass_cut(weights, target_mass);
  if (uncut && cut < 0 && static_cast<int>(weights.size()) < vocab) {
    weights = top_candidates(logits, vocab, penalty, 0);
    for (Candidate& c : weights) c.value = std::exp(c.value * scale - peak);
    cut = mass_cut(weights, target_mass);
  }
  if (cut >= 0) weights.resize(cut);
  const float threshold = min_p * weights[0].value;
  std::vector<Candidate> kept;
  for (const Candidate& c : weights)
    if (c.value >= threshold) kept.push_back(c);
  float mass = 0.0f;
  for (const Candidate& c : kept) mass += c.value;
  const double target = uniform * static_cast<double>(mass);
  double running = 0.0;
  for (const Candidate& c : kept) {
    running += static_cast<double>(c.value);
    if (target < running) return c.id;
  }
  return kept.back().id;  // only through rounding at the last candidate
}

Sampler::Sampler(const SamplerConfig& config) : config_(config), rng_(config.seed) {
  config_.validate();
}

uint32_t Sampler::sample(const float* logits, int vocab, const int32_t* recent, int recent_count) {
  Penalty penalty(config_, recent, recent_count);
  if (config_.temperature == 0.0f) return draw_greedy(logits, vocab, penalty);
  return draw_temperature(logits, vocab, penalty, config_.temperature, config_.top_k,
                          config_.top_p, config_.min_p, rng_.next_f64());
}

}  // namespace vipera
