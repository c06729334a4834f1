#include "cache_manager.hpp"

#include <algorithm>
#include <limits>
#include <string>

namespace vipera {

CacheManager::CacheManager(std::vector<GroupConfig> groups, int num_state_slots, bool reuse) {
  if (num_state_slots <= 0) throw InvalidArgument("a cache needs at least one state slot");
  for (const GroupConfig& config : groups) {
    if (config.page_size <= 0) throw InvalidArgument("page size must be at least 1 token");
    if (config.num_pages <= 0) throw InvalidArgument("a group needs at least one page");
    if (config.window < 0) throw InvalidArgument("a window cannot be negative");
    Group group;
    group.config = config;
    group.refs.assign(config.num_pages, 0);
    // Reverse order on the stack, so that the lowest page number is handed out first
    // (crates/vipera-runtime/src/kv.rs:261-264).
    group.free.reserve(config.num_pages);
    for (int page = config.num_pages - 1; page >= 0; --page) group.free.push_back(page);
    groups_.push_back(std::move(group));
  }
  slot_owner_.assign(num_state_slots, -1);
  for (int slot = num_state_slots - 1; slot >= 0; --slot) free_slots_.push_back(slot);
  // Shared prefixes need pages that are never given back early and one page size for all groups.
  reuse_ = reuse && !groups_.empty();
  for (const Group& group : groups_)
    if (group.config.window > 0 || group.config.page_size != groups_[0].config.page_size) reuse_ = false;
}

// ---------------------------------------------------------------------------------------
// shared prefixes
// ---------------------------------------------------------------------------------------
uint64_t CacheManager::chain_key(uint64_t parent, const int32_t* tokens, int count) {
  uint64_t value = parent ^ 0xCBF29CE484222325ull;
  for (int i = 0; i < count; ++i) {
    value ^= static_cast<uint32_t>(tokens[i]);
    value *= 0x100000001B3ull;
    value ^= value >> 29;
  }
  return value ? value : 1;  // 0 stands for "no prefix"
}

bool CacheManager::unheld(const Kept& kept) const {
  for (size_t g = 0; g < groups_.size(); ++g)
    if (groups_[g].refs[kept.pages[g]] != 1) return false;
  return true;
}

int CacheManager::evictable_pages() const {
  if (evictable_cache_ >= 0) return evictable_cache_;
  // A published page can be given up when no request holds it and every page published
  // behind it can be given up too (they go first).  Deepest pages are looked at first.
  std::vector<std::pair<uint64_t, const Kept*>> order;
  order.reserve(kept_.size());
  for (const auto& item : kept_) order.emplace_back(item.first, &item.second);
  std::sort(order.begin(), order.end(),
            [](const std::pair<uint64_t, const Kept*>& a, const std::pair<uint64_t, const Kept*>& b) {
              return a.second->depth > b.second->depth;
            });
  std::map<uint64_t, int> blocked;  // key -> children that stay
  int count = 0;
  for (const auto& item : order) {
    const Kept& kept = *item.second;
    const bool goes = unheld(kept) && blocked[item.first] == 0;
    if (goes) ++count; else if (kept.parent) ++blocked[kept.parent];
  }
  evictable_cache_ = count;
  return count;
}

void CacheManager::release_page(Group& group, int32_t page) {
  if (--group.refs[page] == 0) group.free.push_back(page);
}

bool CacheManager::evict_one() {
  auto victim = kept_.end();
  for (auto it = kept_.begin(); it != kept_.end(); ++it) {
    if (it->second.children != 0 || !unheld(it->second)) continue;
    if (victim == kept_.end() || it->second.tick < victim->second.tick ||
        (it->second.tick == victim->second.tick && it->second.depth > victim->second.depth))
      victim = it;
  }
  if (victim == kept_.end()) return false;
  for (size_t g = 0; g < groups_.size(); ++g) release_page(groups_[g], victim->second.pages[g]);
  auto parent = kept_.find(victim->second.parent);
  if (victim->second.parent && parent != kept_.end()) --parent->second.children;
  kept_.erase(victim);
  evictable_cache_ = -1;
  return true;
}

int CacheManager::match(int64_t request, const int32_t* tokens, int length) {
  Request& entry = find(request);
  if (!reuse_ || length <= 1) return 0;
  if (entry.computed != 0) throw InvalidArgument("a prefix is matched before anything of the request is computed");
  const int ps = groups_[0].config.page_size;
  const int most = (length - 1) / ps;  // at least one token stays to be computed
  uint64_t key = 0;
  int pages = 0;
  ++tick_;
  for (; pages < most; ++pages) {
    const uint64_t next = chain_key(key, tokens + pages * ps, ps);
    auto found = kept_.find(next);
    if (found == kept_.end() || found->second.parent != key || found->second.depth != pages ||
        !std::equal(found->second.tokens.begin(), found->second.tokens.end(), tokens + pages * ps))
      break;
    found->second.tick = tick_;
    for (size_t g = 0; g < groups_.size(); ++g) {
      entry.tables[g].push_back(found->second.pages[g]);
      ++groups_[g].refs[found->second.pages[g]];
    }
    key = next;
  }
  entry.computed = pages * ps;
  entry.published = pages;
  entry.chain = key;
  if (pages) evictable_cache_ = -1;
  return entry.computed;
}

void CacheManager::publish(int64_t request, const int32_t* tokens, int upto) {
  Request& entry = find(request);
  if (!reuse_) return;
  const int ps = groups_[0].config.page_size;
  const int full = std::min(upto, entry.computed) / ps;
  while (entry.published < full) {
    const int page = entry.published;
    const uint64_t key = chain_key(entry.chain, tokens + page * ps, ps);
    auto found = kept_.find(key);
    if (found == kept_.end()) {
      Kept kept;
      kept.parent = entry.chain;
      kept.depth = page;
      kept.tick = ++tick_;
      kept.tokens.assign(tokens + page * ps, tokens + (page + 1) * ps);
      for (size_t g = 0; g < groups_.size(); ++g) {
        kept.pages.push_back(entry.tables[g].at(page));
        ++groups_[g].refs[entry.tables[g][page]];
      }
      auto parent = kept_.find(entry.chain);
      if (entry.chain && parent != kept_.end()) ++parent->second.children;
      // a parent that was given up meanwhile: this page cannot be reached by a match until
      // the parent is published again; it is given up like any other
      if (entry.chain && parent == kept_.end()) kept.parent = entry.chain;
      kept_.emplace(key, std::move(kept));
      evictable_cache_ = -1;
    } else if (found->second.parent != entry.chain || found->second.depth != page ||
               !std::equal(found->second.tokens.begin(), found->second.tokens.end(), tokens + page * ps)) {
      break;  // two prefixes under one key: the first one stays, this request publishes no further
    } else {
      found->second.tick = ++tick_;
    }
    entry.chain = key;
    ++entry.published;
  }
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
  const int extra = kept_.empty() ? 0 : evictable_pages();  // published pages nobody holds can be taken
  for (size_t g = 0; g < groups_.size(); ++g)
    if (missing[g] > static_cast<int>(groups_[g].free.size()) + extra) return false;
  return true;
}

bool CacheManager::admits(int length, int portion) const {
  for (const Group& group : groups_) {
    const int ps = group.config.page_size;
    int tokens = length;
    if (group.config.window > 0) tokens = std::min(length, group.config.window + portion + ps);
    const int pages = (tokens + ps - 1) / ps;
    const int extra = kept_.empty() ? 0 : evictable_pages();
    if (pages > static_cast<int>(group.free.size()) + extra) return false;
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
  // published pages that nobody holds make room first, least recently used first
  for (size_t g = 0; g < groups_.size(); ++g)
    while (missing[g] > static_cast<int>(groups_[g].free.size()) && evict_one()) {
    }
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
      group.refs[physical] = 1;
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
      release_page(group, table[page]);
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
      release_page(group, table[page]);
    }
  }
  evictable_cache_ = -1;
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
  for (const auto& item : kept_)
    if (group.refs[item.second.pages.at(g)] == 1) ++out.kept_pages;
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
    const std::string where = "group " + std::to_string(g) + ": ";
    std::vector<int> free_seen(group.config.num_pages, 0), holders(group.config.num_pages, 0);
    for (int32_t page : group.free) {
      if (page < 0 || page >= group.config.num_pages)
        return where + "free stack holds page " + std::to_string(page) + " outside the pool";
      if (++free_seen[page] > 1) return where + "page " + std::to_string(page) + " is on the free stack twice";
      if (group.refs[page] != 0) return where + "page " + std::to_string(page) + " is free and marked held";
    }
    for (const auto& item : requests_) {
      std::vector<int> mine(group.config.num_pages, 0);
      for (int32_t page : item.second.tables[g]) {
        if (page < 0) continue;
        if (page >= group.config.num_pages)
          return where + "request " + std::to_string(item.first) + " holds page " + std::to_string(page) + " outside the pool";
        if (++mine[page] > 1)
          return where + "request " + std::to_string(item.first) + " holds page " + std::to_string(page) + " twice";
        ++holders[page];
      }
    }
    std::vector<int> published(group.config.num_pages, 0);
    for (const auto& item : kept_) {
      const int32_t page = item.second.pages.at(g);
      if (page < 0 || page >= group.config.num_pages) return where + "a published page lies outside the pool";
      if (++published[page] > 1) return where + "page " + std::to_string(page) + " is published twice";
      ++holders[page];
    }
    for (int page = 0; page < group.config.num_pages; ++page) {
      if (free_seen[page] && holders[page])
        return where + "page " + std::to_string(page) + " is held twice or held and free";
      if (!free_seen[page] && holders[page] == 0)
        return where + "page " + std::to_string(page) + " is lost (neither free nor held)";
      if (holders[page] != group.refs[page])
        return where + "page " + std::to_string(page) + " is counted " + std::to_string(group.refs[page]) +
               " times and held " + std::to_string(holders[page]) + " times";
      // only a published page may be in more than one table
      if (holders[page] > 1 && !published[page])
        return where + "page " + std::to_string(page) + " is held twice without being published";
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
