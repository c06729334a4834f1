// Python face of the native runtime: cache manager, scheduler, host sampler.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "cache_manager.hpp"
#include "sampler.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace vipera;

namespace {

py::object g_infeasible, g_invalid, g_internal;

template <typename T>
py::array_t<T> to_array(const std::vector<T>& values) {
  py::array_t<T> out(static_cast<py::ssize_t>(values.size()));
  if (!values.empty()) std::memcpy(out.mutable_data(), values.data(), values.size() * sizeof(T));
  return out;
}

SamplerConfig sampler_config_from(const py::dict& d) {
  SamplerConfig c;
  if (d.contains("temperature")) c.temperature = d["temperature"].cast<float>();
  if (d.contains("top_k")) c.top_k = d["top_k"].cast<int>();
  if (d.contains("top_p")) c.top_p = d["top_p"].cast<float>();
  if (d.contains("min_p")) c.min_p = d["min_p"].cast<float>();
  if (d.contains("repetition_penalty")) c.repetition_penalty = d["repetition_penalty"].cast<float>();
  if (d.contains("presence_penalty")) c.presence_penalty = d["presence_penalty"].cast<float>();
  if (d.contains("frequency_penalty")) c.frequency_penalty = d["frequency_penalty"].cast<float>();
  if (d.contains("seed")) c.seed = d["seed"].cast<uint64_t>();
  if (d.contains("logit_bias") && !d["logit_bias"].is_none())
    for (auto item : d["logit_bias"]) {
      auto pair = item.cast<std::pair<uint32_t, float>>();
      c.logit_bias.push_back(pair);
    }
  return c;
}

RequestParams request_params_from(const py::dict& d) {
  RequestParams p;
  p.sampler = sampler_config_from(d);
  if (d.contains("max_new_tokens")) p.max_new_tokens = d["max_new_tokens"].cast<int>();
  if (d.contains("eos_ids") && !d["eos_ids"].is_none())
    p.eos_ids = d["eos_ids"].cast<std::vector<int32_t>>();
  if (d.contains("recent_window")) p.recent_window = d["recent_window"].cast<int>();
  return p;
}

py::dict finished_to_dict(const Finished& f) {
  py::dict d;
  d["request"] = f.request;
  d["reason"] = f.reason;
  d["tokens"] = f.tokens;
  d["prompt_tokens"] = f.prompt_tokens;
  d["processed_tokens"] = f.processed_tokens;
  d["reused_tokens"] = f.reused_tokens;
  d["preemptions"] = f.preemptions;
  return d;
}

py::dict outcome_to_dict(const StepOutcome& o) {
  py::dict d;
  d["tokens"] = o.tokens;
  py::list finished;
  for (const Finished& f : o.finished) finished.append(finished_to_dict(f));
  d["finished"] = finished;
  return d;
}

const float* logits_ptr(const py::array_t<float, py::array::c_style | py::array::forcecast>& a) {
  if (a.ndim() != 1) throw InvalidArgument("logits must be one row of 32-bit floats");
  return a.data();
}

}  // namespace

PYBIND11_MODULE(_vipera_runtime, m) {
  m.doc() = "Native runtime of the engine: paged cache bookkeeping, scheduler, host sampler";

  m.def("_set_error_types", [](py::object infeasible, py::object invalid, py::object internal) {
    g_infeasible = infeasible;
    g_invalid = invalid;
    g_internal = internal;
  });
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const Infeasible& e) {
      PyErr_SetString(g_infeasible ? g_infeasible.ptr() : PyExc_RuntimeError, e.what());
    } catch (const InvalidArgument& e) {
      PyErr_SetString(g_invalid ? g_invalid.ptr() : PyExc_ValueError, e.what());
    } catch (const SampleError& e) {
      PyErr_SetString(g_internal ? g_internal.ptr() : PyExc_RuntimeError, e.what());
    }
  });

  // ---- cache manager ---------------------------------------------------------------
  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init([](const std::vector<std::tuple<int, int, int>>& groups, int slots, bool reuse) {
             std::vector<GroupConfig> configs;
             for (const auto& g : groups) {
               GroupConfig c;
               c.page_size = std::get<0>(g);
               c.num_pages = std::get<1>(g);
               c.window = std::get<2>(g);
               configs.push_back(c);
             }
             return new CacheManager(configs, slots, reuse);
           }),
           py::arg("groups"), py::arg("num_state_slots"), py::arg("reuse") = false)
      .def_property_readonly("reuse", &CacheManager::reuse)
      .def("match", [](CacheManager& c, int64_t request, const std::vector<int32_t>& tokens) {
        return c.match(request, tokens.data(), static_cast<int>(tokens.size()));
      })
      .def("publish", [](CacheManager& c, int64_t request, const std::vector<int32_t>& tokens, int upto) {
        if (upto > static_cast<int>(tokens.size())) throw InvalidArgument("publish beyond the tokens given");
        c.publish(request, tokens.data(), upto);
      })
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def_property_readonly("num_state_slots", &CacheManager::num_state_slots)
      .def_property_readonly("free_state_slots", &CacheManager::free_state_slots)
      .def("group", [](const CacheManager& c, int g) {
        const GroupConfig& config = c.group(g);
        return py::make_tuple(config.page_size, config.num_pages, config.window);
      })
      .def("open", &CacheManager::open)
      .def("is_open", &CacheManager::is_open)
      .def("pages_missing", &CacheManager::pages_missing)
      .def("fits", &CacheManager::fits)
      .def("admits", &CacheManager::admits)
      .def("longest_fit", &CacheManager::longest_fit)
      .def("reserve", &CacheManager::reserve)
      .def("commit", &CacheManager::commit)
      .def("close", &CacheManager::close)
      .def("computed", &CacheManager::computed)
      .def("state_slot", &CacheManager::state_slot)
      .def("table", [](const CacheManager& c, int64_t request, int g) { return to_array(c.table(request, g)); })
      .def("could_ever_fit", &CacheManager::could_ever_fit)
      .def("capacity_tokens", &CacheManager::capacity_tokens)
      .def("stats", [](const CacheManager& c, int g) {
        GroupStats s = c.stats(g);
        py::dict d;
        d["total_pages"] = s.total_pages;
        d["free_pages"] = s.free_pages;
        d["used_pages"] = s.used_pages;
        d["kept_pages"] = s.kept_pages;
        return d;
      })
      .def("open_requests", &CacheManager::open_requests)
      .def("audit", &CacheManager::audit)
      // The inputs of a decode step (every entry one token, every token's logits wanted), written
      // into a host buffer the caller owns (pinned staging memory) in the layout of the captured
      // graphs: [tokens b][positions b][token entry b][entry starts b + 1][first positions b]
      // [state slots b][fresh b][wanted rows b][block table of group g, b x widths[g]] ..., b being
      // the graph's entry count.  Entries past the step's own repeat its first entry.  The
      // constant parts (token entry, entry starts, wanted rows) are the caller's.  Returns the
      // number of entries, or -1 when the step is not of that kind; raises for a step no path
      // may run.
      .def("fill_decode",
           [](const CacheManager& c, const std::vector<int64_t>& requests, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens,
              py::array_t<int32_t, py::array::c_style | py::array::forcecast> counts, py::array_t<int32_t, py::array::c_style | py::array::forcecast> pos0,
              py::array_t<int32_t, py::array::c_style | py::array::forcecast> fresh, py::array_t<int32_t, py::array::c_style | py::array::forcecast> rows,
              uintptr_t host, int bucket, const std::vector<int>& widths, int vocab, int max_model_len) -> int {
             const int n = static_cast<int>(requests.size());
             if (n == 0 || n > bucket) throw InvalidArgument("a decode step needs between one entry and the graph's entry count");
             if (counts.size() != n || pos0.size() != n || fresh.size() != n)
               throw InvalidArgument("requests, counts and first positions must have one item per entry");
             if (tokens.size() != n || rows.size() != n) return -1;
             const int32_t* tok = tokens.data();
             const int32_t* cnt = counts.data();
             const int32_t* pos = pos0.data();
             const int32_t* fr = fresh.data();
             const int32_t* row = rows.data();
             for (int i = 0; i < n; ++i) {
               if (cnt[i] != 1 || row[i] != i) return -1;
             }
             if (static_cast<int>(widths.size()) != c.num_groups()) throw InvalidArgument("one table width is needed for each group");
             int32_t* out = reinterpret_cast<int32_t*>(host);
             const size_t b = static_cast<size_t>(bucket);
             int32_t* out_tokens = out;
             int32_t* out_positions = out + b;
             int32_t* out_pos0 = out + 4 * b + 1;
             int32_t* out_slots = out + 5 * b + 1;
             int32_t* out_fresh = out + 6 * b + 1;
             int32_t* out_tables = out + 8 * b + 1;
             for (int i = 0; i < n; ++i) {
               if (tok[i] < 0 || tok[i] >= vocab) throw InvalidArgument("token id outside the vocabulary of " + std::to_string(vocab));
               if (pos[i] < 0 || pos[i] + 1 > max_model_len)
                 throw InvalidArgument("request " + std::to_string(requests[i]) + ": position " + std::to_string(pos[i]) +
                                       " exceeds the limit of " + std::to_string(max_model_len));
             }
             for (size_t i = 0; i < b; ++i) {
               const int from = i < static_cast<size_t>(n) ? static_cast<int>(i) : 0;
               out_tokens[i] = tok[from];
               out_positions[i] = pos[from];
               out_pos0[i] = pos[from];
               out_slots[i] = c.state_slot(requests[from]);
               out_fresh[i] = fr[from];
             }
             for (int g = 0; g < c.num_groups(); ++g) {
               const int width = widths[g];
               const int page_size = c.group(g).page_size;
               for (size_t i = 0; i < b; ++i) {
                 const int from = i < static_cast<size_t>(n) ? static_cast<int>(i) : 0;
                 const std::vector<int32_t>& table = c.table(requests[from], g);
                 if (static_cast<int>(table.size()) > width) throw InvalidArgument("a block table is longer than the width asked for");
                 const int page = pos[from] / page_size;
                 if (page >= static_cast<int>(table.size()) || table[page] < 0)
                   throw InvalidArgument("a request of the step has no page reserved for its position");
                 int32_t* dst = out_tables + i * width;
                 for (int k = 0; k < width; ++k) dst[k] = k < static_cast<int>(table.size()) ? table[k] : -1;
               }
               out_tables += b * width;
             }
             return n;
           })
      // Block tables of several requests as one [len(requests), width] int32 array; logical
      // pages a request does not hold are -1.
      .def("tables", [](const CacheManager& c, const std::vector<int64_t>& requests, int g, int width) {
        py::array_t<int32_t> out({static_cast<py::ssize_t>(requests.size()), static_cast<py::ssize_t>(width)});
        int32_t* data = out.mutable_data();
        for (size_t r = 0; r < requests.size(); ++r) {
          const std::vector<int32_t>& table = c.table(requests[r], g);
          if (static_cast<int>(table.size()) > width)
            throw InvalidArgument("a block table is longer than the width asked for");
          for (int i = 0; i < width; ++i)
            data[r * width + i] = i < static_cast<int>(table.size()) ? table[i] : -1;
        }
        return out;
      });

  // ---- scheduler -------------------------------------------------------------------
  py::class_<StepPlan>(m, "StepPlan")
      .def_property_readonly("empty", &StepPlan::empty)
      .def_property_readonly("num_entries", [](const StepPlan& p) { return p.entries.size(); })
      .def_property_readonly("num_tokens", [](const StepPlan& p) { return p.tokens.size(); })
      .def_property_readonly("tokens", [](const StepPlan& p) { return to_array(p.tokens); })
      .def_property_readonly("positions", [](const StepPlan& p) { return to_array(p.positions); })
      .def_property_readonly("preempted", [](const StepPlan& p) { return p.preempted; })
      .def_property_readonly("requests", [](const StepPlan& p) {
        std::vector<int64_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.request);
        return v;
      })
      .def_property_readonly("starts", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.start);
        return to_array(v);
      })
      .def_property_readonly("counts", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.count);
        return to_array(v);
      })
      .def_property_readonly("state_slots", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.state_slot);
        return to_array(v);
      })
      .def_property_readonly("fresh", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.fresh ? 1 : 0);
        return to_array(v);
      })
      .def_property_readonly("wants_logits", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const StepEntry& e : p.entries) v.push_back(e.wants_logits ? 1 : 0);
        return to_array(v);
      })
      .def_property_readonly("num_rows", [](const StepPlan& p) { return p.rows.size(); })
      .def_property_readonly("row_requests", [](const StepPlan& p) {
        std::vector<int64_t> v;
        for (const SampleRow& r : p.rows) v.push_back(r.request);
        return v;
      })
      .def_property_readonly("row_token_index", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const SampleRow& r : p.rows) v.push_back(r.token_index);
        return to_array(v);
      })
      .def_property_readonly("row_temperature", [](const StepPlan& p) {
        std::vector<float> v;
        for (const SampleRow& r : p.rows) v.push_back(r.temperature);
        return to_array(v);
      })
      .def_property_readonly("row_top_k", [](const StepPlan& p) {
        std::vector<int32_t> v;
        for (const SampleRow& r : p.rows) v.push_back(r.top_k);
        return to_array(v);
      })
      .def_property_readonly("row_top_p", [](const StepPlan& p) {
        std::vector<float> v;
        for (const SampleRow& r : p.rows) v.push_back(r.top_p);
        return to_array(v);
      })
      .def_property_readonly("row_min_p", [](const StepPlan& p) {
        std::vector<float> v;
        for (const SampleRow& r : p.rows) v.push_back(r.min_p);
        return to_array(v);
      })
      .def_property_readonly("row_uniform", [](const StepPlan& p) {
        std::vector<double> v;
        for (const SampleRow& r : p.rows) v.push_back(r.uniform);
        return to_array(v);
      })
      .def_property_readonly("all_greedy", [](const StepPlan& p) {
        for (const SampleRow& r : p.rows)
          if (r.temperature != 0.0f) return false;
        return true;
      })
      .def_property_readonly("any_penalty", [](const StepPlan& p) {
        for (const SampleRow& r : p.rows)
          if (!r.penalty_ids.empty() || !r.logit_bias.empty()) return true;
        return false;
      })
      // Penalties of one row: (ids, counts, repetition, presence, frequency, bias pairs).
      .def("row_penalty", [](const StepPlan& p, size_t i) {
        const SampleRow& r = p.rows.at(i);
        return py::make_tuple(to_array(r.penalty_ids), to_array(r.penalty_counts), r.repetition_penalty,
                              r.presence_penalty, r.frequency_penalty, r.logit_bias);
      });

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init([](CacheManager* cache, int max_num_seqs, int max_tokens_per_step, int max_portion,
                       int max_model_len, bool reuse_prefixes) {
             SchedulerConfig config;
             config.reuse_prefixes = reuse_prefixes;
             config.max_num_seqs = max_num_seqs;
             config.max_tokens_per_step = max_tokens_per_step;
             config.max_portion = max_portion;
             config.max_model_len = max_model_len;
             return new Scheduler(cache, config);
           }),
           py::arg("cache"), py::arg("max_num_seqs"), py::arg("max_tokens_per_step"),
           py::arg("max_portion"), py::arg("max_model_len") = 0, py::arg("reuse_prefixes") = true,
           py::keep_alive<1, 2>())
      .def("add", [](Scheduler& s, int64_t request, std::vector<int32_t> prompt, const py::dict& params) {
        s.add(request, std::move(prompt), request_params_from(params));
      })
      .def("cancel", &Scheduler::cancel)
      .def("has_work", &Scheduler::has_work)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def("schedule", &Scheduler::schedule)
      .def("plan_ahead", &Scheduler::plan_ahead, py::arg("plan"), py::arg("max_top_k") = 0)
      .def("peek_uniforms", [](const Scheduler& s, const StepPlan& plan) { return to_array(s.peek_uniforms(plan)); })
      .def("complete", [](Scheduler& s, const StepPlan& plan, const std::vector<int32_t>& sampled) {
        return outcome_to_dict(s.complete(plan, sampled));
      })
      .def("fail", [](Scheduler& s, const StepPlan& plan) { return outcome_to_dict(s.fail(plan)); });

  // ---- host sampler ----------------------------------------------------------------
  py::class_<Rng>(m, "Rng")
      .def(py::init<uint64_t>(), py::arg("seed") = 0)
      .def("reseed", &Rng::reseed)
      .def("next_u64", &Rng::next_u64)
      .def("next_f64", &Rng::next_f64);

  py::class_<Sampler>(m, "Sampler")
      .def(py::init([](const py::dict& d) {
        SamplerConfig config = sampler_config_from(d);
        try {
          config.validate();
        } catch (const std::invalid_argument& e) {
          throw InvalidArgument(e.what());
        }
        return new Sampler(config);
      }))
      .def("sample", [](Sampler& s, py::array_t<float, py::array::c_style | py::array::forcecast> logits,
                        const std::vector<int32_t>& recent) {
        return s.sample(logits_ptr(logits), static_cast<int>(logits.shape(0)), recent.data(),
                        static_cast<int>(recent.size()));
      }, py::arg("logits"), py::arg("recent") = std::vector<int32_t>());

  m.def("draw_greedy", [](py::array_t<float, py::array::c_style | py::array::forcecast> logits,
                          const py::dict& config, const std::vector<int32_t>& recent) {
    SamplerConfig c = sampler_config_from(config);
    Penalty penalty(c, recent.data(), static_cast<int>(recent.size()));
    return draw_greedy(logits_ptr(logits), static_cast<int>(logits.shape(0)), penalty);
  }, py::arg("logits"), py::arg("config") = py::dict(), py::arg("recent") = std::vector<int32_t>());

  m.def("draw_temperature", [](py::array_t<float, py::array::c_style | py::array::forcecast> logits,
                               const py::dict& config, const std::vector<int32_t>& recent, double uniform) {
    SamplerConfig c = sampler_config_from(config);
    Penalty penalty(c, recent.data(), static_cast<int>(recent.size()));
    return draw_temperature(logits_ptr(logits), static_cast<int>(logits.shape(0)), penalty, c.temperature,
                            c.top_k, c.top_p, c.min_p, uniform);
  }, py::arg("logits"), py::arg("config"), py::arg("recent"), py::arg("uniform"));

  m.attr("NO_CUT_CANDIDATES") = kNoCutCandidates;
}
