// Host-side accounting of the paged cache: pages, block tables, state slots.
//
// The reference's BlockManager (crates/core/engine/src/blocks/manager.rs:130-135)
// keeps one uniform pool for all layers. Here layers with the same needs form a
// group, and every group has pages and block tables of its own: a group either
// keeps every position (window == 0) or only the last `window` positions, whose
// older pages go back to the free list as soon as the window has passed them.
// The protocol per step is the reference's (crates/core/engine/src/blocks.rs:17-45):
// reserve (all or nothing) -> the forward pass writes -> commit.
// Beside the pages every request holds one slot of fixed-size state.
//
// Pages are counted by reference, as the reference's blocks are
// (manager.rs:614-628): fork() lets a new request start from everything
// another has computed. The pages that are full are shared (a request only
// ever writes at and beyond its own computed positions, so a full page is
// never written again); the partly filled last page is copied for the child
// (the reference's copy-on-write of a partial tail, manager.rs:749-763), which
// the caller does on the device from the list fork() returns.
#pragma once

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace mxb {

struct GroupConfig {
  int page_tokens = 16;  // positions per page
  int window = 0;        // 0: every position is kept; else the last `window`
  int num_pages = 0;     // pages of this group's pool
};

// Raised when a reservation does not fit; the manager is unchanged
// (manager.rs:484-490: OutOfBlocks{needed, free}).
struct OutOfPages : public std::runtime_error {
  int group, needed, free;
  OutOfPages(int group_, int needed_, int free_)
      : std::runtime_error("out of cache pages: group " + std::to_string(group_) + " needs " +
                           std::to_string(needed_) + ", " + std::to_string(free_) + " free"),
        group(group_), needed(needed_), free(free_) {}
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupConfig> groups, int max_requests)
      : groups_(std::move(groups)), max_requests_(max_requests) {
    if (max_requests_ <= 0) throw std::invalid_argument("max_requests must be positive");
    for (const GroupConfig& g : groups_) {
      if (g.page_tokens <= 0) throw std::invalid_argument("page_tokens must be positive");
      if (g.window < 0) throw std::invalid_argument("window must not be negative");
      if (g.num_pages < 0) throw std::invalid_argument("num_pages must not be negative");
    }
    free_pages_.resize(groups_.size());
    refs_.resize(groups_.size());
    ever_used_.resize(groups_.size());
    for (size_t g = 0; g < groups_.size(); ++g) {
      // Last-in first-out: the page given back last is handed out first, so a
      // small pool reuses pages at once.
      for (int p = groups_[g].num_pages - 1; p >= 0; --p) free_pages_[g].push_back(p);
      refs_[g].assign(groups_[g].num_pages, 0);
      ever_used_[g].assign(groups_[g].num_pages, false);
    }
    for (int s = max_requests_ - 1; s >= 0; --s) free_slots_.push_back(s);
  }

  int num_groups() const { return static_cast<int>(groups_.size()); }
  const GroupConfig& group(int g) const { return groups_.at(g); }
  int max_requests() const { return max_requests_; }
  int free_pages(int g) const { return static_cast<int>(free_pages_.at(g).size()); }
  int free_slots() const { return static_cast<int>(free_slots_.size()); }
  int live_requests() const { return static_cast<int>(requests_.size()); }
  bool has(int64_t id) const { return requests_.count(id) != 0; }
  uint64_t pages_handed_out() const { return pages_handed_out_; }
  uint64_t pages_reused() const { return pages_reused_; }

  // Gives the request a state slot. It holds no pages yet.
  int admit(int64_t id) {
    if (has(id)) throw std::invalid_argument("request " + std::to_string(id) + " is already live");
    if (free_slots_.empty()) throw std::runtime_error("no free request slot");
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.epoch = ++admissions_;
    r.tables.resize(groups_.size());
    r.first_live.assign(groups_.size(), 0);
    requests_.emplace(id, std::move(r));
    return requests_.at(id).slot;
  }

  int slot(int64_t id) const { return get(id).slot; }
  // Counts admissions: an id that was released and admitted again has a new
  // epoch, so whoever mirrors its table knows the mirror is stale.
  uint64_t epoch(int64_t id) const { return get(id).epoch; }
  int64_t reserved(int64_t id) const { return get(id).reserved; }
  int64_t computed(int64_t id) const { return get(id).computed; }

  // Pages each group would have to hand out for `tokens` more positions of
  // `id`; an unknown id is costed as a new request.
  std::vector<int> cost(int64_t id, int64_t tokens) const {
    std::vector<int> out(groups_.size(), 0);
    auto it = requests_.find(id);
    int64_t reserved = it == requests_.end() ? 0 : it->second.reserved;
    for (size_t g = 0; g < groups_.size(); ++g) {
      int64_t held = it == requests_.end() ? 0 : static_cast<int64_t>(it->second.tables[g].size());
      int64_t want = ceil_div(reserved + tokens, groups_[g].page_tokens);
      out[g] = static_cast<int>(want > held ? want - held : 0);
    }
    return out;
  }

  // Whether all of `asks` (id, tokens) fit together right now.
  bool fits(const std::vector<std::pair<int64_t, int64_t>>& asks) const {
    std::vector<int64_t> need(groups_.size(), 0);
    for (const auto& ask : asks) {
      std::vector<int> c = cost(ask.first, ask.second);
      for (size_t g = 0; g < groups_.size(); ++g) need[g] += c[g];
    }
    for (size_t g = 0; g < groups_.size(); ++g)
      if (need[g] > free_pages(static_cast<int>(g))) return false;
    return true;
  }

  // Reserves positions reserved .. reserved+tokens-1 in every group, or
  // throws OutOfPages and changes nothing.
  void reserve(int64_t id, int64_t tokens) {
    if (tokens <= 0) throw std::invalid_argument("reserve needs a positive token count");
    Request& r = get(id);
    std::vector<int> need = cost(id, tokens);
    for (size_t g = 0; g < groups_.size(); ++g)
      if (need[g] > free_pages(static_cast<int>(g)))
        throw OutOfPages(static_cast<int>(g), need[g], free_pages(static_cast<int>(g)));
    for (size_t g = 0; g < groups_.size(); ++g) {
      for (int n = 0; n < need[g]; ++n) {
        r.tables[g].push_back(take_page(static_cast<int>(g)));
      }
    }
    r.reserved += tokens;
  }

  // Marks `tokens` reserved positions as written, then gives back the pages of
  // windowed groups that no later query can see.
  void commit(int64_t id, int64_t tokens) {
    Request& r = get(id);
    if (tokens < 0 || r.computed + tokens > r.reserved)
      throw std::invalid_argument("commit beyond the reserved positions");
    r.computed += tokens;
    for (size_t g = 0; g < groups_.size(); ++g) {
      const GroupConfig& cfg = groups_[g];
      if (cfg.window == 0) continue;
      // The next query sits at position >= computed and sees keys
      // > position - window, so keys below computed - window + 1 are dead.
      int64_t first_needed = r.computed - cfg.window + 1;
      if (first_needed <= 0) continue;
      int64_t dead_pages = first_needed / cfg.page_tokens;  // pages wholly below
      for (int64_t p = r.first_live[g]; p < dead_pages && p < static_cast<int64_t>(r.tables[g].size()); ++p) {
        give_back(static_cast<int>(g), r.tables[g][p]);
        r.tables[g][p] = -1;
      }
      if (dead_pages > r.first_live[g])
        r.first_live[g] = std::min<int64_t>(dead_pages, static_cast<int64_t>(r.tables[g].size()));
    }
  }

  // Drops positions that were reserved but not committed (a failed step).
  void rollback(int64_t id) {
    Request& r = get(id);
    bool shrank = false;
    for (size_t g = 0; g < groups_.size(); ++g) {
      int64_t keep = ceil_div(r.computed, groups_[g].page_tokens);
      while (static_cast<int64_t>(r.tables[g].size()) > keep) {
        int page = r.tables[g].back();
        r.tables[g].pop_back();
        if (page >= 0) give_back(static_cast<int>(g), page);
        shrank = true;
      }
    }
    r.reserved = r.computed;
    if (shrank) r.epoch = ++admissions_;  // a mirror of the longer table is stale now
  }

  // Everything the request holds goes back: pages last-first, then the slot
  // (manager.rs:639-648).
  void release(int64_t id) {
    Request& r = get(id);
    for (size_t g = 0; g < groups_.size(); ++g)
      for (auto it = r.tables[g].rbegin(); it != r.tables[g].rend(); ++it)
        if (*it >= 0) give_back(static_cast<int>(g), *it);
    free_slots_.push_back(r.slot);
    requests_.erase(id);
  }

  // What the device has to copy after a fork: the partly filled last page of
  // each group (`group`, from page `source` to page `target`) and the state slot.
  struct PageCopy {
    int group, source, target;
  };
  struct Fork {
    int source_slot = -1, target_slot = -1;
    std::vector<PageCopy> copies;
  };

  // A new request `child` that holds everything `parent` has computed: it
  // shares the parent's full pages and gets a page of its own for the partly
  // filled last one. All or nothing: throws OutOfPages (or for a lack of
  // slots) and changes nothing. The parent must have no uncommitted positions.
  Fork fork(int64_t parent, int64_t child) {
    if (has(child)) throw std::invalid_argument("request " + std::to_string(child) + " is already live");
    const Request& from = get(parent);
    if (from.reserved != from.computed) throw std::invalid_argument("fork of a request with uncommitted positions");
    if (free_slots_.empty()) throw std::runtime_error("no free request slot");
    for (size_t g = 0; g < groups_.size(); ++g) {
      const bool partial = from.computed % groups_[g].page_tokens != 0 && !from.tables[g].empty() &&
                           from.tables[g].back() >= 0;
      if (partial && free_pages(static_cast<int>(g)) < 1) throw OutOfPages(static_cast<int>(g), 1, 0);
    }
    Fork out;
    Request r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.epoch = ++admissions_;
    r.reserved = r.computed = from.computed;
    r.first_live = from.first_live;
    r.tables = from.tables;
    out.source_slot = from.slot;
    out.target_slot = r.slot;
    for (size_t g = 0; g < groups_.size(); ++g) {
      const int64_t full = from.computed / groups_[g].page_tokens;   // pages no one writes again
      for (size_t p = 0; p < r.tables[g].size(); ++p) {
        const int page = r.tables[g][p];
        if (page < 0) continue;
        if (static_cast<int64_t>(p) < full) {
          ++refs_[g][page];
        } else {
          r.tables[g][p] = take_page(static_cast<int>(g));
          out.copies.push_back({static_cast<int>(g), page, r.tables[g][p]});
        }
      }
    }
    requests_.emplace(child, std::move(r));
    return out;
  }

  // How many requests hold a page (0: it is free).
  int references(int g, int page) const { return refs_.at(g).at(page); }

  // Logical page -> physical page of one group, -1 where the window has
  // passed the page.
  const std::vector<int>& table(int64_t id, int g) const { return get(id).tables.at(g); }
  int64_t first_live_page(int64_t id, int g) const { return get(id).first_live.at(g); }

  std::vector<int64_t> live_ids() const {
    std::vector<int64_t> out;
    for (const auto& kv : requests_) out.push_back(kv.first);
    return out;
  }

  // Every page is free exactly once, or held by as many requests as its
  // reference count says and not free; every slot is free or held exactly
  // once (manager.rs:658-714 checks the same for blocks).
  void check_invariants() const {
    for (size_t g = 0; g < groups_.size(); ++g) {
      std::vector<int> free_count(groups_[g].num_pages, 0), held(groups_[g].num_pages, 0);
      for (int page : free_pages_[g]) {
        if (page < 0 || page >= groups_[g].num_pages) throw std::logic_error("free page out of range");
        if (refs_[g][page] != 0) throw std::logic_error("a free page is still referred to");
        if (++free_count[page] > 1) throw std::logic_error("a page is free twice");
      }
      for (const auto& kv : requests_) {
        const Request& r = kv.second;
        std::vector<int> own(groups_[g].num_pages, 0);
        for (size_t p = 0; p < r.tables[g].size(); ++p) {
          int page = r.tables[g][p];
          if (page < 0) {
            if (static_cast<int64_t>(p) >= r.first_live[g]) throw std::logic_error("a hole inside the live pages");
            continue;
          }
          if (page >= groups_[g].num_pages) throw std::logic_error("held page out of range");
          if (++own[page] > 1) throw std::logic_error("a request holds a page twice");
          if (free_count[page]) throw std::logic_error("a page is held and free");
          ++held[page];
          // a page that is shared lies wholly below what its holders have computed
          if (refs_[g][page] > 1 && static_cast<int64_t>(p + 1) * groups_[g].page_tokens > r.computed)
            throw std::logic_error("a shared page can still be written");
        }
        if (static_cast<int64_t>(r.tables[g].size()) != ceil_div(r.reserved, groups_[g].page_tokens))
          throw std::logic_error("table length does not match the reserved positions");
        if (r.computed > r.reserved) throw std::logic_error("computed beyond reserved");
      }
      for (int page = 0; page < groups_[g].num_pages; ++page) {
        if (held[page] != refs_[g][page]) throw std::logic_error("a page's reference count is off");
        if (held[page] == 0 && free_count[page] != 1) throw std::logic_error("a page is lost");
      }
    }
    std::vector<int> slots(max_requests_, 0);
    for (int s : free_slots_) ++slots.at(s);
    for (const auto& kv : requests_) ++slots.at(kv.second.slot);
    for (int s = 0; s < max_requests_; ++s)
      if (slots[s] != 1) throw std::logic_error("a state slot is lost or held twice");
  }

 private:
  struct Request {
    int slot = -1;
    uint64_t epoch = 0;
    int64_t reserved = 0;  // positions with a page slot
    int64_t computed = 0;  // positions whose keys and values are written
    std::vector<std::vector<int>> tables;  // [group][logical page]
    std::vector<int64_t> first_live;       // [group] first logical page still held
  };

  static int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

  Request& get(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw std::invalid_argument("unknown request " + std::to_string(id));
    return it->second;
  }
  const Request& get(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw std::invalid_argument("unknown request " + std::to_string(id));
    return it->second;
  }

  int take_page(int g) {
    int page = free_pages_[g].back();
    free_pages_[g].pop_back();
    if (refs_[g][page] != 0) throw std::logic_error("a free page is still referred to");
    refs_[g][page] = 1;
    if (ever_used_[g][page]) ++pages_reused_;
    ever_used_[g][page] = true;
    ++pages_handed_out_;
    return page;
  }

  // One holder less; the page is free again when nobody holds it.
  void give_back(int g, int page) {
    if (refs_[g][page] <= 0) throw std::logic_error("a page is freed that nobody holds");
    if (--refs_[g][page] == 0) free_pages_[g].push_back(page);
  }

  std::vector<GroupConfig> groups_;
  int max_requests_;
  std::vector<std::vector<int>> free_pages_;
  std::vector<std::vector<int>> refs_;   // [group][page] requests that hold the page
  std::vector<std::vector<bool>> ever_used_;
  std::vector<int> free_slots_;
  std::unordered_map<int64_t, Request> requests_;
  uint64_t pages_handed_out_ = 0, pages_reused_ = 0, admissions_ = 0;
};

}  // namespace mxb
