#include "cache_manager.hpp"

#include <algorithm>
#include <limits>
#include <string>

namespace vipera {

CacheManager::CacheManager(std::vector<GroupConfig> groups, int num_state_slots) {
  if (num_state_slots <= 0) throw InvalidArgument("a cache needs at least one state slot");
  for (const GroupConfig& config : groups) {
    if (config.page_size <= 0) throw InvalidArgument("page size must be at least 1 token");
    if (config.num_pages <= 0) throw InvalidArgument("a group needs at least one page");
    if (config.window < 0) throw InvalidArgument("a window cannot be negative");
    Group group;
    group.config = config;
    group.held.assign(config.num_pages, 0);
    // Reverse order on the stack, so that the lowest page number is handed out first
    // (crates/vipera-runtime/src/kv.rs:261-264).
    group.free.reserve(config.num_pages);
    for (int page = config.num_pages - 1; page >= 0; --page) group.free.push_back(page);
    groups_.push_back(std::move(group));
  }
  slot_owner_.assign(num_state_slots, -1);
  for (int slot = num_state_slots - 1; slot >= 0; --slot) free_slots_.push_back(slot);
}

const CacheManager::Request& CacheManager::find(int64_t request) const {
  auto it = requests_.find(request);
  if (it == requests_.end())
    throw InvalidArgument("request " + std::to_string(request) + " is not open in the cache");
  return it->second;
}

CacheManager::Request& CacheManager::find(int64_t request) {
  return const_cast<Request&>(static_cast<const CacheManager*>(this)->find(request));
}

int CacheManager::open(int64_t request) {
  if (requests_.count(request))
    throw InvalidArgument("request " + std::to_string(request) + " is already open in the cache");
  if (free_slots_.empty())
    throw Infeasible("no state slot is free for request " + std::to_string(request));
  Request entry;
  entry.slot = free_slots_.back();
  free_slots_.pop_back();
  slot_owner_[entry.slot] = request;
  entry.tables.resize(groups_.size());
  requests_.emplace(request, std::move(entry));
  return requests_[request].slot;
}

void CacheManager::span(const GroupConfig& config, int computed, int new_length, int* first,
                        int* end) {
  const int ps = config.page_size;
  int oldest = 0;
  if (config.window > 0) oldest = std::max(0, computed - config.window + 1);
  *first = oldest / ps;
  *end = (new_length + ps - 1) / ps;
}

std::vector<int> CacheManager::pages_missing(int64_t request, int new_length) const {
  const Request& entry = find(request);
  if (new_length < entry.computed)
    throw InvalidArgument("a request cannot shrink below the tokens already computed");
  std::vector<int> missing(groups_.size(), 0);
  for (size_t g = 0; g < groups_.size(); ++g) {
    int first, end;
    span(groups_[g].config, entry.computed, new_length, &first, &end);
    const std::vector<int32_t>& table = entry.tables[g];
    for (int page = first; page < end; ++page)
      if (page >= static_cast<int>(table.size()) || table[page] < 0) ++missing[g];
  }
  return missing;
}

bool CacheManager::fits(int64_t request, int new_length) const {
  std::vector<int> missing = pages_missing(request, new_length);
  for (size_t g = 0; g < groups_.size(); ++g)
    if (missing[g] > static_cast<int>(groups_[g].free.size())) return false;
  return true;
}

bool CacheManager::admits(int length, int portion) const {
  for (const Group& group : groups_) {
    const int ps = group.config.page_size;
    int tokens = length;
    if (group.config.window > 0) tokens = std::min(length, group.config.window + portion + ps);
    const int pages = (tokens + ps - 1) / ps;
    if (pages > static_cast<int>(group.free.size())) return false;
  }
  return true;
}

int CacheManager::longest_fit(int64_t request, int new_length) const {
  const Request& entry = find(request);
  int low = entry.computed, high = new_length;  // `low` always fits: it needs nothing new
  if (fits(request, high)) return high;
  while (high - low > 1) {
    int middle = low + (high - low) / 2;
    if (fits(request, middle)) low = middle; else high = middle;
  }
  return low;
}

void CacheManager::reserve(int64_t request, int new_length) {
  std::vector<int> missing = pages_missing(request, new_length);
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (missing[g] > static_cast<int>(groups_[g].free.size())) {
      // (plain string building: stream formatting has crashed inside processes that load
      // several C++ runtimes)
      throw Infeasible("cache is full: " + std::to_string(missing[g]) + " pages needed for request " +
                       std::to_string(request) + " in group " + std::to_string(g) + ", " +
                       std::to_string(groups_[g].free.size()) + " free");
    }
  }
  Request& entry = find(request);
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& group = groups_[g];
    int first, end;
    span(group.config, entry.computed, new_length, &first, &end);
    std::vector<int32_t>& table = entry.tables[g];
    if (static_cast<int>(table.size()) < end) table.resize(end, -1);
    for (int page = first; page < end; ++page) {
      if (table[page] >= 0) continue;
      int32_t physical = group.free.back();
      group.free.pop_back();
      group.held[physical] = 1;
      table[page] = physical;
    }
  }
}

void CacheManager::commit(int64_t request, int new_length) {
  Request& entry = find(request);
  if (new_length < entry.computed)
    throw InvalidArgument("commit cannot move a request backwards");
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupConfig& config = groups_[g].config;
    const std::vector<int32_t>& table = entry.tables[g];
    int end = (new_length + config.page_size - 1) / config.page_size;
    int first, unused;
    span(config, entry.computed, new_length, &first, &unused);
    for (int page = first; page < end; ++page)
      if (page >= static_cast<int>(table.size()) || table[page] < 0)
        throw InvalidArgument("commit of tokens whose pages were never reserved");
  }
  entry.computed = new_length;
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& group = groups_[g];
    if (group.config.window <= 0) continue;
    // The next query stands at `new_length` or later and reads keys from
    // new_length - window + 1 on; pages wholly before that are out of every reach.
    int oldest = std::max(0, new_length - group.config.window + 1);
    int keep_from = oldest / group.config.page_size;
    std::vector<int32_t>& table = entry.tables[g];
    for (int page = 0; page < keep_from && page < static_cast<int>(table.size()); ++page) {
      if (table[page] < 0) continue;
      group.held[table[page]] = 0;
      group.free.push_back(table[page]);
      table[page] = -1;
    }
  }
}

void CacheManager::close(int64_t request) {
  Request& entry = find(request);
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& group = groups_[g];
    // Tail first, so that the lowest page of the request is handed out next
    // (crates/vipera-runtime/src/kv.rs:374-379 returns blocks the same way).
    std::vector<int32_t>& table = entry.tables[g];
    for (int page = static_cast<int>(table.size()) - 1; page >= 0; --page) {
      if (table[page] < 0) continue;
      group.held[table[page]] = 0;
      group.free.push_back(table[page]);
    }
  }
  slot_owner_[entry.slot] = -1;
  free_slots_.push_back(entry.slot);
  requests_.erase(request);
}

int CacheManager::computed(int64_t request) const { return find(request).computed; }
int CacheManager::state_slot(int64_t request) const { return find(request).slot; }

const std::vector<int32_t>& CacheManager::table(int64_t request, int g) const {
  return find(request).tables.at(g);
}

bool CacheManager::could_ever_fit(int length) const { return length <= capacity_tokens(); }

int64_t CacheManager::capacity_tokens() const {
  int64_t best = std::numeric_limits<int64_t>::max();
  for (const Group& group : groups_) {
    if (group.config.window > 0) {
      // A windowed group holds window + one portion; it bounds nothing as long as it
      // has the pages for the window itself and one page more.
      int64_t least = (group.config.window + group.config.page_size - 1) / group.config.page_size + 1;
      if (group.config.num_pages < least) best = std::min<int64_t>(best, 0);
      continue;
    }
    best = std::min<int64_t>(best, int64_t(group.config.num_pages) * group.config.page_size);
  }
  return best;
}

GroupStats CacheManager::stats(int g) const {
  const Group& group = groups_.at(g);
  GroupStats out;
  out.total_pages = group.config.num_pages;
  out.free_pages = static_cast<int>(group.free.size());
  out.used_pages = out.total_pages - out.free_pages;
  return out;
}

std::vector<int64_t> CacheManager::open_requests() const {
  std::vector<int64_t> ids;
  for (const auto& item : requests_) ids.push_back(item.first);
  return ids;
}

std::string CacheManager::audit() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const Group& group = groups_[g];
    std::vector<int> seen(group.config.num_pages, 0);
    for (int32_t page : group.free) {
      if (page < 0 || page >= group.config.num_pages) {
        return std::string("group ") + std::to_string(g) + std::string(": free stack holds page ") + std::to_string(page) + std::string(" outside the pool");
      }
      if (++seen[page] > 1) {
        return std::string("group ") + std::to_string(g) + std::string(": page ") + std::to_string(page) + std::string(" is on the free stack twice");
      }
      if (group.held[page]) {
        return std::string("group ") + std::to_string(g) + std::string(": page ") + std::to_string(page) + std::string(" is free and marked held");
      }
    }
    for (const auto& item : requests_) {
      for (int32_t page : item.second.tables[g]) {
        if (page < 0) continue;
        if (page >= group.config.num_pages) {
          return std::string("group ") + std::to_string(g) + std::string(": request ") + std::to_string(item.first) + std::string(" holds page ") + std::to_string(page) + std::string(" outside the pool");
        }
        if (++seen[page] > 1) {
          return std::string("group ") + std::to_string(g) + std::string(": page ") + std::to_string(page) + std::string(" is held twice or held and free");
        }
        if (!group.held[page]) {
          return std::string("group ") + std::to_string(g) + std::string(": page ") + std::to_string(page) + std::string(" is in a table but not marked held");
        }
      }
    }
    for (int page = 0; page < group.config.num_pages; ++page) {
      if (seen[page] == 0) {
        return std::string("group ") + std::to_string(g) + std::string(": page ") + std::to_string(page) + std::string(" is lost (neither free nor held)");
      }
    }
  }
  std::vector<int> slots(slot_owner_.size(), 0);
  for (int slot : free_slots_) {
    if (++slots.at(slot) > 1) return "state slot " + std::to_string(slot) + " is free twice";
    if (slot_owner_[slot] != -1) return "state slot " + std::to_string(slot) + " is free and owned";
  }
  for (const auto& item : requests_) {
    if (++slots.at(item.second.slot) > 1)
      return "state slot " + std::to_string(item.second.slot) + " is held twice";
    if (slot_owner_[item.second.slot] != item.first)
      return "state slot " + std::to_string(item.second.slot) + " has the wrong owner";
  }
  for (size_t slot = 0; slot < slots.size(); ++slot)
    if (slots[slot] == 0) return "state slot " + std::to_string(slot) + " is lost";
  return "";
}

}  // namespace vipera
