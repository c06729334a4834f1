// Host-side sampling: the generator, the penalties and the two strategies.
//
// Behaviour follows the reference's sampler crate: xorshift64* seeded through
// SplitMix64 (crates/vipera-sampler/src/rng.rs:13-57); greedy = best penalised finite
// logit, ties to the lowest id (crates/vipera-sampler/src/lib.rs:135-156); temperature =
// penalty, bounded best-first head, softmax mass over every finite logit, top-p cut on a
// share of that mass, min-p filter against the best weight, one draw (lib.rs:172-247);
// penalties as in lib.rs:596-616.  The device sampler is held to this one in the tests,
// and the engine falls back to it for the one case the device kernel does not cover (no
// top-k cut and a top-p head longer than the bounded head).
#pragma once

#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

namespace vipera {

struct SampleError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// How many candidates are kept when top_k is 0 before every logit has to be sorted
// (crates/vipera-sampler/src/lib.rs:437).
constexpr int kNoCutCandidates = 4096;

class Rng {
 public:
  explicit Rng(uint64_t seed = 0) { reseed(seed); }
  void reseed(uint64_t seed);
  uint64_t next_u64();
  double next_f64();  // uniform in [0, 1)
  uint64_t state() const { return state_; }

 private:
  uint64_t state_ = 0;
};

struct SamplerConfig {
  float temperature = 0.8f;  // 0 selects greedy and skips every other filter
  int top_k = 40;            // 0: no cut
  float top_p = 0.95f;
  float min_p = 0.05f;
  float repetition_penalty = 1.0f;
  float presence_penalty = 0.0f;
  float frequency_penalty = 0.0f;
  std::vector<std::pair<uint32_t, float>> logit_bias;  // at most 16 entries
  uint64_t seed = 0;

  void validate() const;  // throws std::invalid_argument with the reference's wording
  bool has_penalty() const {
    return repetition_penalty != 1.0f || presence_penalty != 0.0f || frequency_penalty != 0.0f ||
           !logit_bias.empty();
  }
};

// Counts of recent tokens and the biases, both sorted by id.
class Penalty {
 public:
  Penalty() = default;
  Penalty(const SamplerConfig& config, const int32_t* recent, int recent_count);
  float apply(uint32_t id, float logit) const;
  bool empty() const { return counts_.empty() && bias_.empty(); }
  // Every id that apply() changes, ascending, with its count (0 for a bias-only id).
  const std::vector<std::pair<uint32_t, uint32_t>>& counts() const { return counts_; }
  const std::vector<std::pair<uint32_t, float>>& bias() const { return bias_; }

 private:
  std::vector<std::pair<uint32_t, uint32_t>> counts_;
  std::vector<std::pair<uint32_t, float>> bias_;
  float factor_ = 1.0f, presence_ = 0.0f, frequency_ = 0.0f;
};

uint32_t draw_greedy(const float* logits, int vocab, const Penalty& penalty);
// `uniform` is the generator's next_f64(), passed in so that the same draw can be
// given to the device kernel.
uint32_t draw_temperature(const float* logits, int vocab, const Penalty& penalty, float temperature,
                          int top_k, float top_p, float min_p, double uniform);

// Config + generator, one per request: the same seed gives the same tokens whatever else
// is in the batch (crates/vipera-runtime/src/engine.rs:612).
class Sampler {
 public:
  explicit Sampler(const SamplerConfig& config);
  uint32_t sample(const float* logits, int vocab, const int32_t* recent, int recent_count);
  const SamplerConfig& config() const { return config_; }
  Rng& rng() { return rng_; }

 private:
  SamplerConfig config_;
  Rng rng_;
};

}  // namespace vipera
