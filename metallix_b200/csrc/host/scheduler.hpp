// Continuous batching above the step function: admits requests, cuts prompts
// into portions under a token budget, decodes, finishes and frees.
//
// The decisions follow the reference's engine loop
// (crates/app/cli/src/engine_loop.rs): a waiting queue in arrival order and a
// running list in admission order (:484-508); admission keeps one page of
// headroom per running request while anything runs, and an idle engine admits
// regardless (:823-861); every running request decodes one token per iteration
// (:931-967); when pages run out, a request that is still in its prompt goes
// first, else the one admitted last, it gives back its pages and returns to
// the FRONT of the waiting queue with everything it has produced, to be
// computed again later (:1138-1167, :440-457); a lone request that cannot grow
// fails. Unlike the reference, whose prompt portions are sized by a time
// budget (:398-423) and run as forward passes of their own, portions here are
// sized in tokens and ride in the same step as the decoded tokens.
#pragma once

#include <cstdint>
#include <deque>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "cache_manager.hpp"

namespace mxb {

struct Limits {
  int max_num_seqs = 8;            // requests that run together at most
  int max_tokens_per_step = 8192;  // tokens of one step, decoded ones included
  int prefill_chunk = 0;           // most prompt tokens of one request per step; 0: no cap
};

struct SamplingParams {
  double temperature = 0.0;  // 0: greedy
  uint64_t seed = 0;
  double top_p = 1.0;
  int top_k = 0;   // 0: off
  int sampler = 0; // 0: inverse CDF, 1: race (Gumbel-max)
};

struct RequestInfo {
  int64_t id = -1;
  std::vector<int32_t> prompt;
  std::vector<int32_t> output;
  int max_new_tokens = 0;
  std::vector<int32_t> stop_ids;
  bool ignore_eos = false;
  SamplingParams sampling;
  int preemptions = 0;
  std::string finish_reason;  // "", "eos", "length", "cancelled", "deadline", or an error text
  bool failed = false;
  double deadline = 0.0;      // on the caller's clock, seconds; 0: none
};

struct PlanEntry {
  int64_t id;
  int64_t start;                // position of tokens[0]
  std::vector<int32_t> tokens;  // the portion this step runs
  bool wants_token;             // the portion reaches the end: sample after it
  int generated_position;       // index of the token to sample (for the RNG)
};

struct StepPlan {
  std::vector<PlanEntry> entries;
  std::vector<int64_t> preempted;  // requests that gave their pages back
  std::vector<int64_t> failed;     // requests that can never run
  int decode_tokens = 0, prefill_tokens = 0;
};

struct Event {
  int64_t id;
  int32_t token;
  bool finished;
  std::string finish_reason;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, Limits limits) : cache_(cache), limits_(limits) {
    if (limits_.max_num_seqs <= 0 || limits_.max_tokens_per_step <= 0)
      throw std::invalid_argument("scheduler limits must be positive");
    if (limits_.max_num_seqs > cache_->max_requests())
      throw std::invalid_argument("max_num_seqs exceeds the cache manager's request slots");
  }

  int64_t add(std::vector<int32_t> prompt, int max_new_tokens, std::vector<int32_t> stop_ids,
              bool ignore_eos, SamplingParams sampling, double deadline = 0.0) {
    if (prompt.empty()) throw std::invalid_argument("a request needs at least one prompt token");
    if (max_new_tokens <= 0) throw std::invalid_argument("max_new_tokens must be positive");
    RequestInfo r;
    r.id = next_id_++;
    r.prompt = std::move(prompt);
    r.max_new_tokens = max_new_tokens;
    r.stop_ids = std::move(stop_ids);
    r.ignore_eos = ignore_eos;
    r.sampling = sampling;
    r.deadline = deadline;
    int64_t id = r.id;
    requests_.emplace(id, std::move(r));
    waiting_.push_back(id);
    return id;
  }

  // A cancelled request leaves at the next plan() (engine_loop.rs:631-653).
  void cancel(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end() || !it->second.finish_reason.empty()) return;
    cancelled_.push_back(id);
  }

  bool idle() const { return waiting_.empty() && running_.empty(); }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  const RequestInfo& request(int64_t id) const { return requests_.at(id); }
  const std::vector<int64_t>& running() const { return running_; }
  std::vector<int64_t> waiting() const { return std::vector<int64_t>(waiting_.begin(), waiting_.end()); }
  void forget(int64_t id) { requests_.erase(id); }

  // Decides the next step. Changes the cache manager only by releasing
  // preempted, cancelled or failed requests and by admitting (a slot, no
  // pages); the step function reserves the pages the plan was costed for.
  // `now`: the caller's clock, for the requests that have a deadline: one whose
  // deadline has passed leaves as a cancelled one does, whether it waits, is
  // in its prompt or decodes (engine_loop.rs:631-653, :932-943).
  StepPlan plan(double now = 0.0) {
    StepPlan plan;
    drop_cancelled();
    drop_overdue(now);
    for (;;) {
      plan_once(plan);
      if (!plan.entries.empty() || running_.empty()) break;
      // Requests hold pages but none can move: the one admitted last (one
      // still in its prompt first) makes room, or fails if it is alone.
      std::vector<int64_t> claimed(cache_->num_groups(), 0);
      int64_t victim = pick_victim(plan);
      if (running_.size() == 1) fail(victim, "the sequence outgrew the KV pool", plan);
      else preempt(victim, plan, claimed);
    }
    return plan;
  }

  // Takes the tokens picked for the plan's entries that wanted one (same
  // order), appends them, finishes and frees (engine_loop.rs:901-911).
  std::vector<Event> update(const StepPlan& plan, const std::vector<int32_t>& tokens) {
    std::vector<Event> events;
    size_t next = 0;
    for (const PlanEntry& e : plan.entries) {
      if (!e.wants_token) continue;
      if (next >= tokens.size()) throw std::invalid_argument("fewer tokens than the plan wanted");
      int32_t token = tokens[next++];
      RequestInfo& r = requests_.at(e.id);
      r.output.push_back(token);
      bool stop = false;
      if (!r.ignore_eos)
        for (int32_t s : r.stop_ids) stop = stop || s == token;
      std::string reason;
      if (stop) reason = "eos";  // crates/app/cli/src/qwen_forward.rs:968-974
      else if (static_cast<int>(r.output.size()) >= r.max_new_tokens) reason = "length";
      if (!reason.empty()) finish(e.id, reason);
      events.push_back(Event{e.id, token, !reason.empty(), reason});
    }
    if (next != tokens.size()) throw std::invalid_argument("more tokens than the plan wanted");
    return events;
  }

  // A step that failed after the plan was made: every request of the plan
  // leaves with the error (crates/models/qwen/src/forward/paged.rs:776-781).
  void fail_plan(const StepPlan& plan, const std::string& why) {
    for (const PlanEntry& e : plan.entries) {
      RequestInfo& r = requests_.at(e.id);
      if (!r.finish_reason.empty()) continue;
      r.failed = true;
      finish(e.id, why);
    }
  }

 private:
  bool is_running(int64_t id) const {
    for (int64_t r : running_)
      if (r == id) return true;
    return false;
  }

  void plan_once(StepPlan& plan) {
    std::vector<int64_t> claimed(cache_->num_groups(), 0);  // pages this plan will take
    int budget = limits_.max_tokens_per_step;

    // 1. One token for every request that is past its prompt.
    std::vector<int64_t> snapshot = running_;
    for (int64_t id : snapshot) {
      if (budget == 0) break;
      if (!is_running(id) || pending(id) != 1 || cache_->computed(id) == 0) continue;
      bool gone = false;
      while (!fits(id, 1, claimed)) {
        // Pages ran out in the middle of decoding.
        int64_t victim = pick_victim(plan);
        if (running_.size() == 1) {
          fail(id, "the sequence outgrew the KV pool", plan);
          gone = true;
          break;
        }
        preempt(victim, plan, claimed);
        if (victim == id) { gone = true; break; }
      }
      if (gone) continue;
      claim(id, 1, claimed);
      plan.entries.push_back(make_entry(id, 1));
      plan.decode_tokens += 1;
      budget -= 1;
    }

    // 2. Portions of prompts that are already admitted, in admission order.
    snapshot = running_;
    for (int64_t id : snapshot) {
      if (!is_running(id) || in_plan(plan, id)) continue;
      int64_t want = portion(id, budget);
      while (want > 0 && !fits(id, want, claimed)) want = shrink(id, want, claimed);
      if (want == 0) continue;
      claim(id, want, claimed);
      plan.entries.push_back(make_entry(id, want));
      plan.prefill_tokens += static_cast<int>(want);
      budget -= static_cast<int>(want);
    }

    // 3. Admission in arrival order.
    while (!waiting_.empty() && static_cast<int>(running_.size()) < limits_.max_num_seqs && budget > 0) {
      int64_t id = waiting_.front();
      int64_t context = context_len(id);
      if (!running_.empty()) {
        if (!admits(id, context, claimed)) break;
      } else if (!cache_->fits({{id, context}})) {
        // An idle engine admits regardless, and the request fails at once if
        // the whole pool cannot hold it (engine_loop.rs:776-781).
        waiting_.pop_front();
        fail(id, "the prompt does not fit the KV pool", plan);
        continue;
      }
      int64_t want = portion(id, budget);
      while (want > 0 && !fits(id, want, claimed)) want = shrink(id, want, claimed);
      if (want == 0) break;
      waiting_.pop_front();
      cache_->admit(id);
      running_.push_back(id);
      claim(id, want, claimed);
      plan.entries.push_back(make_entry(id, want));
      plan.prefill_tokens += static_cast<int>(want);
      budget -= static_cast<int>(want);
    }
  }

  int64_t context_len(int64_t id) const {
    const RequestInfo& r = requests_.at(id);
    return static_cast<int64_t>(r.prompt.size() + r.output.size());
  }
  int64_t computed_of(int64_t id) const { return cache_->has(id) ? cache_->computed(id) : 0; }
  int64_t pending(int64_t id) const { return context_len(id) - computed_of(id); }

  int64_t portion(int64_t id, int budget) const {
    int64_t want = pending(id);
    if (limits_.prefill_chunk > 0 && want > limits_.prefill_chunk) want = limits_.prefill_chunk;
    if (want > budget) want = budget;
    return want;
  }

  bool fits(int64_t id, int64_t tokens, const std::vector<int64_t>& claimed) const {
    std::vector<int> c = cache_->cost(id, tokens);
    for (int g = 0; g < cache_->num_groups(); ++g)
      if (claimed[g] + c[g] > cache_->free_pages(g)) return false;
    return true;
  }

  // The admission rule: the whole context must fit beside one page of
  // headroom for every running request (engine_loop.rs:823-861).
  bool admits(int64_t id, int64_t context, const std::vector<int64_t>& claimed) const {
    std::vector<int> c = cache_->cost(id, context);
    for (int g = 0; g < cache_->num_groups(); ++g)
      if (claimed[g] + c[g] + static_cast<int64_t>(running_.size()) > cache_->free_pages(g)) return false;
    return true;
  }

  void claim(int64_t id, int64_t tokens, std::vector<int64_t>& claimed) const {
    std::vector<int> c = cache_->cost(id, tokens);
    for (int g = 0; g < cache_->num_groups(); ++g) claimed[g] += c[g];
  }

  // The largest portion below `want` that ends on a page boundary of the
  // tightest group, or 0.
  int64_t shrink(int64_t id, int64_t want, const std::vector<int64_t>& claimed) const {
    int64_t start = cache_->has(id) ? cache_->reserved(id) : 0;
    int64_t best = 0;
    for (int g = 0; g < cache_->num_groups(); ++g) {
      int64_t room = cache_->free_pages(g) - claimed[g];
      if (room < 0) room = 0;
      int64_t held = cache_->has(id) ? static_cast<int64_t>(cache_->table(id, g).size()) : 0;
      int64_t reach = (held + room) * cache_->group(g).page_tokens - start;  // tokens that fit
      if (g == 0 || reach < best) best = reach;
    }
    if (best >= want) best = want - 1;
    return best > 0 ? best : 0;
  }

  PlanEntry make_entry(int64_t id, int64_t tokens) const {
    const RequestInfo& r = requests_.at(id);
    int64_t start = computed_of(id);
    PlanEntry e;
    e.id = id;
    e.start = start;
    for (int64_t p = start; p < start + tokens; ++p)
      e.tokens.push_back(p < static_cast<int64_t>(r.prompt.size())
                             ? r.prompt[p] : r.output[p - static_cast<int64_t>(r.prompt.size())]);
    e.wants_token = start + tokens == context_len(id);
    e.generated_position = static_cast<int>(r.output.size());
    return e;
  }

  static bool in_plan(const StepPlan& plan, int64_t id) {
    for (const PlanEntry& e : plan.entries)
      if (e.id == id) return true;
    return false;
  }

  // A request still in its prompt goes first, else the one admitted last
  // (engine_loop.rs:1138-1167). Requests already in this plan are spared
  // unless nothing else is left.
  int64_t pick_victim(const StepPlan& plan) const {
    for (auto it = running_.rbegin(); it != running_.rend(); ++it)
      if (pending(*it) > 1 && !in_plan(plan, *it)) return *it;
    for (auto it = running_.rbegin(); it != running_.rend(); ++it)
      if (!in_plan(plan, *it)) return *it;
    return running_.back();
  }

  void preempt(int64_t id, StepPlan& plan, std::vector<int64_t>& claimed) {
    // An entry already planned for the victim is withdrawn with its claim.
    for (size_t i = 0; i < plan.entries.size(); ++i) {
      if (plan.entries[i].id != id) continue;
      std::vector<int> c = cache_->cost(id, static_cast<int64_t>(plan.entries[i].tokens.size()));
      for (int g = 0; g < cache_->num_groups(); ++g) claimed[g] -= c[g];
      if (plan.entries[i].tokens.size() == 1 && plan.entries[i].start > 0) plan.decode_tokens -= 1;
      else plan.prefill_tokens -= static_cast<int>(plan.entries[i].tokens.size());
      plan.entries.erase(plan.entries.begin() + static_cast<long>(i));
      break;
    }
    cache_->release(id);
    remove_running(id);
    requests_.at(id).preemptions += 1;
    waiting_.push_front(id);
    plan.preempted.push_back(id);
  }

  void fail(int64_t id, const std::string& why, StepPlan& plan) {
    requests_.at(id).failed = true;
    finish(id, why);
    plan.failed.push_back(id);
  }

  void finish(int64_t id, const std::string& reason) {
    requests_.at(id).finish_reason = reason;
    if (cache_->has(id)) cache_->release(id);
    remove_running(id);
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
      if (*it == id) { waiting_.erase(it); break; }
  }

  void remove_running(int64_t id) {
    for (size_t i = 0; i < running_.size(); ++i)
      if (running_[i] == id) { running_.erase(running_.begin() + static_cast<long>(i)); return; }
  }

  void drop_cancelled() {
    for (int64_t id : cancelled_) {
      auto it = requests_.find(id);
      if (it == requests_.end() || !it->second.finish_reason.empty()) continue;
      finish(id, "cancelled");
    }
    cancelled_.clear();
  }

  void drop_overdue(double now) {
    std::vector<int64_t> overdue;
    for (int64_t id : waiting_)
      if (requests_.at(id).deadline > 0.0 && now >= requests_.at(id).deadline) overdue.push_back(id);
    for (int64_t id : running_)
      if (requests_.at(id).deadline > 0.0 && now >= requests_.at(id).deadline) overdue.push_back(id);
    for (int64_t id : overdue) finish(id, "deadline");
  }

  CacheManager* cache_;
  Limits limits_;
  int64_t next_id_ = 0;
  std::map<int64_t, RequestInfo> requests_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_;
  std::vector<int64_t> cancelled_;
};

}  // namespace mxb
