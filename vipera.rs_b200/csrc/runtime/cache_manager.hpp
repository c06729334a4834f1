// Paged cache bookkeeping: which physical page holds which part of which request.
//
// The reference keeps one pool of fixed-size blocks, a free stack that hands out the
// lowest block first, and a block table per sequence; a reservation either succeeds
// whole or leaves nothing behind (crates/vipera-runtime/src/kv.rs:232-382), and
// release returns every block of a sequence (kv.rs:539-561).  This manager keeps that
// behaviour and adds two things the reference does not have: several groups of layers,
// each with pages of its own and possibly a window after which pages are given back,
// and a pool of fixed-size state slots, one per live request.
//
// Reuse of prompt prefixes.  The reference parks a finished sequence's blocks and copies
// whole blocks of a matching prefix into a new sequence (kv.rs:440-514; engine.rs:432-491:
// prompt positions only, longest common prefix, at least one block, at least one token left
// to compute).  Here pages are shared instead of copied: a full page of a prompt can be
// `publish`ed under the tokens of the whole prefix up to its end; `match` gives a new request
// the published pages of its longest matching prefix (they are counted, not copied, and never
// written again: a request writes from its computed length on, which then is a page
// boundary).  Published pages that no request holds are given up, least recently used first,
// when a reservation needs pages, so reuse never causes a refusal (kv.rs:365-373).  Reuse needs
// groups without windows and with one page size.
//
// Only bookkeeping lives here.  The device memory the page numbers index is owned by
// the Python side; nothing in this file touches a GPU.
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace vipera {

struct Infeasible : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct InvalidArgument : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct GroupConfig {
  int page_size = 16;  // tokens per page
  int num_pages = 0;   // pages in this group's pool
  int window = 0;      // 0: every key is kept; w > 0: a query at p reads keys p-w+1 .. p
};

struct GroupStats {
  int total_pages = 0;
  int free_pages = 0;
  int used_pages = 0;
  int kept_pages = 0;  // published for reuse and held by no request
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupConfig> groups, int num_state_slots, bool reuse = false);

  // Whether prefixes are shared (asked for, and the groups allow it).
  bool reuse() const { return reuse_; }
  // The request (open, nothing computed yet) takes the published pages of the longest prefix
  // of `tokens` that is known, leaving at least one token to compute; returns the number of
  // tokens it need not compute.
  int match(int64_t request, const int32_t* tokens, int length);
  // Full pages of tokens [0, upto) of the request (computed, and a prefix worth sharing: its
  // prompt) become available to later requests.
  void publish(int64_t request, const int32_t* tokens, int upto);

  int num_groups() const { return static_cast<int>(groups_.size()); }
  const GroupConfig& group(int g) const { return groups_.at(g).config; }
  int num_state_slots() const { return static_cast<int>(slot_owner_.size()); }
  int free_state_slots() const { return static_cast<int>(free_slots_.size()); }

  // A request enters: it gets a state slot and empty tables.  Throws Infeasible when no
  // slot is free, InvalidArgument when the id is already open.
  int open(int64_t request);
  bool is_open(int64_t request) const { return requests_.count(request) != 0; }

  // Pages that `reserve(request, new_length)` would have to take, per group.
  std::vector<int> pages_missing(int64_t request, int new_length) const;
  // Whether `reserve(request, new_length)` would succeed now.
  bool fits(int64_t request, int new_length) const;
  // Whether a request of `length` tokens, computed in portions of at most `portion` tokens,
  // can be taken in now: groups that keep every key need pages for all of it, windowed
  // groups for the window and one portion.
  bool admits(int length, int portion) const;
  // The longest length <= new_length that fits now (never below the computed length).
  int longest_fit(int64_t request, int new_length) const;
  // Make sure every page is held that computing tokens [computed, new_length) reads or
  // writes.  All groups or nothing: on failure no table changes and Infeasible is thrown.
  void reserve(int64_t request, int new_length);
  // Tokens [computed, new_length) are now in the cache.  Pages that no later query can
  // read (a window has passed them) go back to the free stack.
  void commit(int64_t request, int new_length);
  // The request leaves: all its pages and its slot are returned.
  void close(int64_t request);

  int computed(int64_t request) const;
  int state_slot(int64_t request) const;
  // Logical page index -> physical page, -1 where no page is held.
  const std::vector<int32_t>& table(int64_t request, int g) const;
  // Whether a request of this many tokens could ever be held, alone, by every group.
  bool could_ever_fit(int length) const;
  // Tokens one request can hold at most (the smallest bound over the groups).
  int64_t capacity_tokens() const;

  GroupStats stats(int g) const;
  std::vector<int64_t> open_requests() const;
  // Consistency of the books: every page is either free or held exactly once.  Returns
  // an empty string when sound, else a description of the first fault found.
  std::string audit() const;

 private:
  struct Group {
    GroupConfig config;
    std::vector<int32_t> free;  // stack; back() is handed out next
    std::vector<int32_t> refs;  // per physical page: tables that hold it, plus one while published
  };
  struct Request {
    int slot = -1;
    int computed = 0;
    std::vector<std::vector<int32_t>> tables;  // per group
    int published = 0;    // pages of this request looked at by publish()
    uint64_t chain = 0;   // key of the prefix that ends with page `published - 1`
  };
  // One published page: the same logical page of every group, under the key of its prefix.
  struct Kept {
    std::vector<int32_t> pages;   // physical page per group
    std::vector<int32_t> tokens;  // the page's own tokens (a key is a hash: equal keys are checked)
    uint64_t parent = 0;
    int depth = 0;      // logical page index
    int children = 0;   // published pages whose prefix runs through this one
    uint64_t tick = 0;  // last use
  };

  // First and one-past-last logical page that computing [computed, new_length) touches.
  static void span(const GroupConfig& config, int computed, int new_length, int* first, int* end);
  const Request& find(int64_t request) const;
  Request& find(int64_t request);

  static uint64_t chain_key(uint64_t parent, const int32_t* tokens, int count);
  bool unheld(const Kept& kept) const;   // no request holds its pages
  int evictable_pages() const;           // published pages a reservation may take
  bool evict_one();                      // give up the least recently used unheld leaf
  void release_page(Group& group, int32_t page);

  std::vector<Group> groups_;
  std::map<uint64_t, Kept> kept_;
  bool reuse_ = false;
  uint64_t tick_ = 0;
  mutable int evictable_cache_ = -1;     // -1: not known
  std::map<int64_t, Request> requests_;
  std::vector<int64_t> slot_owner_;  // -1 when free
  std::vector<int> free_slots_;      // stack; back() is handed out next
};

}  // namespace vipera
