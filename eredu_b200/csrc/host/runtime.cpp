// Host-side runtime state machines (no tensors, no CUDA): parallel topology arithmetic, the paged-KV block
// manager, the fair continuous-batching scheduler and the cross-rank consensus word frames.
//
// Behavioural references: eredu-core/src/topology.rs:65-167,195-387,495-520 (rank formula, ranges,
// ownership); eredu/src/backend/mlx/runtime/distributed/parallel.rs:111-131 (partition units aligned to
// quantisation groups); eredu-core/src/cache/lifecycle.rs:34-330 and cache/policy.rs (leases, protected
// prefix, eviction candidates); eredu-core/src/scheduler.rs:15-1410 (request lifecycle, fairness, bounded
// admission, cancellation, poisoning); eredu-core/src/consensus.rs:12-244 (schedule / completion frames).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace eredu {

// ============================================================================================ topology
static std::pair<int64_t, int64_t> balanced_range(int64_t total, int64_t parts, int64_t index) {
  if (parts <= 0 || index < 0 || index >= parts) throw std::invalid_argument("invalid partition");
  const int64_t base = total / parts, extra = total % parts;
  const int64_t start = index * base + std::min(index, extra);
  return {start, start + base + (index < extra ? 1 : 0)};
}

// Split `total` elements over `parts` ranks in whole `unit`s (a unit = lcm of the structural unit, e.g. a
// GQA group or a SwiGLU pair, and the quantisation group), balanced and contiguous.
static std::vector<std::pair<int64_t, int64_t>> aligned_partition_units(int64_t total, int64_t unit, int64_t parts) {
  if (unit <= 0 || total % unit != 0) throw std::invalid_argument("total is not a multiple of the partition unit");
  const int64_t units = total / unit;
  std::vector<std::pair<int64_t, int64_t>> out;
  for (int64_t r = 0; r < parts; ++r) {
    auto [a, b] = balanced_range(units, parts, r);
    out.emplace_back(a * unit, b * unit);
  }
  return out;
}

// ============================================================================================ block manager
// Pages are 16-token KV slabs. Page 0 is reserved (padding target). Sealed (full, immutable) pages can be
// registered under a content hash for prefix reuse; an unreferenced sealed page stays cached until evicted
// (LRU or LFU). Sequences hold leases (reference counts) on their pages.
class BlockManager {
 public:
  explicit BlockManager(int64_t num_pages, const std::string& eviction = "lru") : num_pages_(num_pages), lfu_(eviction == "lfu") {
    if (num_pages < 2) throw std::invalid_argument("need at least 2 pages");
    refs_.assign(num_pages, 0);
    hash_of_.assign(num_pages, 0);
    has_hash_.assign(num_pages, false);
    uses_.assign(num_pages, 0);
    stamp_.assign(num_pages, 0);
    for (int64_t p = num_pages - 1; p >= 1; --p) free_.push_back(p);
  }

  int64_t free_pages() const { return static_cast<int64_t>(free_.size() + cached_.size()); }
  int64_t num_pages() const { return num_pages_; }
  int64_t cached_pages() const { return static_cast<int64_t>(cached_.size()); }

  std::vector<int64_t> alloc(int64_t n) {
    if (n > free_pages()) throw std::runtime_error("KV pool exhausted: need " + std::to_string(n) + " pages, " + std::to_string(free_pages()) + " free");
    std::vector<int64_t> out;
    for (int64_t i = 0; i < n; ++i) {
      int64_t p;
      if (!free_.empty()) {
        p = free_.back();
        free_.pop_back();
      } else {
        p = evict_one();
      }
      refs_[p] = 1;
      out.push_back(p);
    }
    return out;
  }

  void retain(const std::vector<int64_t>& pages) {
    for (int64_t p : pages) {
      check(p);
      if (refs_[p] == 0) cached_.erase(p);  // revive a cached page
      ++refs_[p];
    }
  }

  void release(const std::vector<int64_t>& pages) {
    for (int64_t p : pages) {
      check(p);
      if (refs_[p] <= 0) throw std::runtime_error("double release of page " + std::to_string(p));
      if (--refs_[p] == 0) {
        if (has_hash_[p]) {
          stamp_[p] = ++clock_;
          cached_.insert(p);
        } else {
          free_.push_back(p);
        }
      }
    }
  }

  // Register a sealed page under the hash of (parent hash, its 16 token ids).
  void seal(int64_t page, uint64_t hash) {
    check(page);
    auto it = by_hash_.find(hash);
    if (it != by_hash_.end() && it->second != page) return;  // an identical page is already published
    by_hash_[hash] = page;
    hash_of_[page] = hash;
    has_hash_[page] = true;
  }

  static uint64_t chain_hash(uint64_t parent, const std::vector<int32_t>& tokens) {
    uint64_t h = parent ^ 0x9E3779B97F4A7C15ull;
    for (int32_t t : tokens) {
      h ^= static_cast<uint64_t>(static_cast<uint32_t>(t)) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
      h *= 0xBF58476D1CE4E5B9ull;
      h ^= h >> 31;
    }
    return h;
  }

  // Longest cached prefix of `tokens` in whole pages: returns the pages (leased to the caller) in order.
  std::vector<int64_t> match_prefix(const std::vector<int32_t>& tokens) {
    std::vector<int64_t> out;
    uint64_t h = 0;
    for (size_t i = 0; i + 16 <= tokens.size(); i += 16) {
      std::vector<int32_t> chunk(tokens.begin() + i, tokens.begin() + i + 16);
      h = chain_hash(h, chunk);
      auto it = by_hash_.find(h);
      if (it == by_hash_.end()) break;
      out.push_back(it->second);
    }
    retain(out);
    for (int64_t p : out) ++uses_[p];
    return out;
  }

  // Publish the full pages of a sequence for prefix reuse: page i holds tokens [16 i, 16 i + 16). Returns the number
  // of pages visited (each is now published under its chained hash, or an identical page already was).
  int64_t seal_prefix(const std::vector<int64_t>& pages, const std::vector<int32_t>& tokens) {
    uint64_t h = 0;
    int64_t n = 0;
    for (size_t i = 0; i + 16 <= tokens.size() && i / 16 < pages.size(); i += 16) {
      std::vector<int32_t> chunk(tokens.begin() + i, tokens.begin() + i + 16);
      h = chain_hash(h, chunk);
      seal(pages[i / 16], h);
      ++n;
    }
    return n;
  }

  int refcount(int64_t page) const { return refs_.at(page); }

  // The page published under `hash` on the device, or -1.
  int64_t lookup(uint64_t hash) const {
    auto it = by_hash_.find(hash);
    return it == by_hash_.end() ? -1 : it->second;
  }

  // (page, hash) of every published page that was evicted to satisfy an allocation since the last call. The page has
  // a new owner already, but its old contents stay in device memory until that owner's first write: a lower tier
  // copies them out before the next forward pass.
  std::vector<std::pair<int64_t, uint64_t>> take_evicted() {
    std::vector<std::pair<int64_t, uint64_t>> out;
    out.swap(evicted_log_);
    return out;
  }

 private:
  void check(int64_t p) const {
    if (p <= 0 || p >= num_pages_) throw std::out_of_range("page id out of range");
  }
  int64_t evict_one() {
    if (cached_.empty()) throw std::runtime_error("no evictable page");
    int64_t best = -1;
    for (int64_t p : cached_) {
      if (best < 0) best = p;
      else if (lfu_ ? (uses_[p] < uses_[best] || (uses_[p] == uses_[best] && stamp_[p] < stamp_[best])) : stamp_[p] < stamp_[best]) best = p;
    }
    cached_.erase(best);
    if (evicted_log_.size() < 65536) evicted_log_.emplace_back(best, hash_of_[best]);
    by_hash_.erase(hash_of_[best]);
    has_hash_[best] = false;
    uses_[best] = 0;
    ++evictions_;
    return best;
  }

  int64_t num_pages_;
  bool lfu_;
  std::vector<int> refs_;
  std::vector<uint64_t> hash_of_;
  std::vector<bool> has_hash_;
  std::vector<int64_t> uses_, stamp_;
  std::vector<int64_t> free_;
  std::set<int64_t> cached_;
  std::unordered_map<uint64_t, int64_t> by_hash_;
  std::vector<std::pair<int64_t, uint64_t>> evicted_log_;
  int64_t clock_ = 0;

 public:
  int64_t evictions_ = 0;
};

// ============================================================================================ scheduler
enum class ReqState { Waiting, Prefilling, Decoding, Finished, Cancelled, Failed };

static const char* state_name(ReqState s) {
  switch (s) {
    case ReqState::Waiting: return "waiting";
    case ReqState::Prefilling: return "prefilling";
    case ReqState::Decoding: return "decoding";
    case ReqState::Finished: return "finished";
    case ReqState::Cancelled: return "cancelled";
    default: return "failed";
  }
}

struct Request {
  uint64_t id;
  int64_t prompt_tokens;
  int64_t max_new_tokens;
  int64_t prefilled = 0;
  int64_t generated = 0;
  double deadline = 0.0;  // 0 = none
  ReqState state = ReqState::Waiting;
  bool cancel_requested = false;
  std::string finish_reason;
  uint64_t in_flight_work = 0;  // nonzero while a submitted step has not been completed
};

struct WorkItem {
  uint64_t work_id;
  uint64_t request_id;
  std::string kind;  // "prefill" | "decode"
  int64_t tokens;
};

// Fair, bounded, transactional: a step plan is built round-robin over runnable requests under the batch and
// token budgets; a request with work in flight is never scheduled again until that work is completed;
// cancellation never pre-empts submitted work (it takes effect when the work completes); any consensus
// mismatch poisons the scheduler and every later call fails closed.
class Scheduler {
 public:
  Scheduler(int64_t max_batch, int64_t max_step_tokens, int64_t max_waiting, int64_t prefill_chunk)
      : max_batch_(max_batch), max_step_tokens_(max_step_tokens), max_waiting_(max_waiting), prefill_chunk_(prefill_chunk) {}

  uint64_t submit(int64_t prompt_tokens, int64_t max_new_tokens, double deadline) {
    fail_if_poisoned();
    if (prompt_tokens <= 0) throw std::invalid_argument("empty prompt");
    if (static_cast<int64_t>(order_.size()) >= max_waiting_ + max_batch_) throw std::runtime_error("admission refused: queue full");
    Request r;
    r.id = next_request_++;
    r.prompt_tokens = prompt_tokens;
    r.max_new_tokens = max_new_tokens;
    r.deadline = deadline;
    reqs_[r.id] = r;
    order_.push_back(r.id);
    ++stats_submitted_;
    return r.id;
  }

  void cancel(uint64_t id) {
    auto& r = get(id);
    if (terminal(r.state)) return;
    if (r.in_flight_work != 0) {
      r.cancel_requested = true;  // cooperative: resolved when the in-flight work completes
      return;
    }
    finish(r, ReqState::Cancelled, "cancelled");
  }

  std::vector<WorkItem> plan_step(double now) {
    fail_if_poisoned();
    std::vector<WorkItem> plan;
    int64_t budget = max_step_tokens_;
    int64_t running = 0;
    for (auto& kv : reqs_)
      if (kv.second.state == ReqState::Prefilling || kv.second.state == ReqState::Decoding) ++running;
    const size_t n = order_.size();
    for (size_t k = 0; k < n && static_cast<int64_t>(plan.size()) < max_batch_ && budget > 0; ++k) {
      const uint64_t id = order_[(cursor_ + k) % n];
      Request& r = reqs_[id];
      if (terminal(r.state) || r.in_flight_work != 0) continue;
      if (r.deadline > 0.0 && now > r.deadline) {
        finish(r, ReqState::Cancelled, "deadline");
        continue;
      }
      if (r.state == ReqState::Waiting) {
        if (running >= max_batch_) continue;
        r.state = ReqState::Prefilling;
        ++running;
      }
      WorkItem w;
      w.work_id = next_work_++;
      w.request_id = id;
      if (r.state == ReqState::Prefilling) {
        w.kind = "prefill";
        w.tokens = std::min({r.prompt_tokens - r.prefilled, prefill_chunk_, budget});
      } else {
        w.kind = "decode";
        w.tokens = 1;
      }
      if (w.tokens <= 0) continue;
      budget -= w.tokens;
      r.in_flight_work = w.work_id;
      plan.push_back(w);
    }
    if (n) cursor_ = (cursor_ + 1) % n;  // rotate the starting point: no request is starved
    ++stats_steps_;
    return plan;
  }

  // Report the outcome of one work item. `generated` = tokens committed by this work (0 for a non-final
  // prefill chunk), `stop` = the request hit EOS / a stop sequence, `failed` = request-local failure.
  std::string complete(uint64_t work_id, int64_t tokens, int64_t generated, bool stop, bool failed) {
    fail_if_poisoned();
    for (auto& kv : reqs_) {
      Request& r = kv.second;
      if (r.in_flight_work != work_id) continue;
      r.in_flight_work = 0;
      if (failed) {
        finish(r, ReqState::Failed, "failed");
      } else {
        if (r.state == ReqState::Prefilling) {
          r.prefilled += tokens;
          if (r.prefilled >= r.prompt_tokens) r.state = ReqState::Decoding;
        }
        r.generated += generated;
        if (r.cancel_requested) finish(r, ReqState::Cancelled, "cancelled");
        else if (stop) finish(r, ReqState::Finished, "stop");
        else if (r.generated >= r.max_new_tokens) finish(r, ReqState::Finished, "max_tokens");
      }
      return state_name(r.state);
    }
    throw std::runtime_error("unknown work id");
  }

  void poison(const std::string& why) {
    poisoned_ = true;
    poison_reason_ = why;
  }
  bool poisoned() const { return poisoned_; }

  py::dict request(uint64_t id) const {
    const Request& r = reqs_.at(id);
    py::dict d;
    d["state"] = state_name(r.state);
    d["prefilled"] = r.prefilled;
    d["generated"] = r.generated;
    d["finish_reason"] = r.finish_reason;
    d["in_flight"] = r.in_flight_work != 0;
    return d;
  }

  py::dict report() const {
    py::dict d;
    int64_t waiting = 0, running = 0, done = 0;
    for (const auto& kv : reqs_) {
      if (kv.second.state == ReqState::Waiting) ++waiting;
      else if (!terminal(kv.second.state)) ++running;
      else ++done;
    }
    d["submitted"] = stats_submitted_;
    d["steps"] = stats_steps_;
    d["waiting"] = waiting;
    d["running"] = running;
    d["finished"] = done;
    d["poisoned"] = poisoned_;
    d["poison_reason"] = poison_reason_;
    return d;
  }

  void reap() {
    std::deque<uint64_t> keep;
    for (uint64_t id : order_)
      if (!terminal(reqs_[id].state)) keep.push_back(id);
      else reqs_.erase(id);
    order_ = keep;
    cursor_ = 0;
  }

 private:
  static bool terminal(ReqState s) { return s == ReqState::Finished || s == ReqState::Cancelled || s == ReqState::Failed; }
  void fail_if_poisoned() const {
    if (poisoned_) throw std::runtime_error("scheduler is poisoned: " + poison_reason_);
  }
  Request& get(uint64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) throw std::out_of_range("unknown request");
    return it->second;
  }
  void finish(Request& r, ReqState s, const std::string& why) {
    r.state = s;
    r.finish_reason = why;
  }

  int64_t max_batch_, max_step_tokens_, max_waiting_, prefill_chunk_;
  std::map<uint64_t, Request> reqs_;
  std::deque<uint64_t> order_;
  size_t cursor_ = 0;
  uint64_t next_request_ = 1, next_work_ = 1;
  bool poisoned_ = false;
  std::string poison_reason_;
  int64_t stats_submitted_ = 0, stats_steps_ = 0;
};

// ============================================================================================ consensus
// Frames are flat u32 words so that any transport that can all-gather integers can carry them.
static std::vector<uint32_t> encode_schedule(const std::vector<std::pair<uint64_t, std::vector<uint32_t>>>& plan,
                                             uint64_t drain_cycle, uint64_t protocol) {
  std::vector<uint32_t> w = {static_cast<uint32_t>(plan.size()), static_cast<uint32_t>(drain_cycle),
                             static_cast<uint32_t>(drain_cycle >> 32), static_cast<uint32_t>(protocol),
                             static_cast<uint32_t>(protocol >> 32)};
  for (const auto& item : plan) {
    w.push_back(static_cast<uint32_t>(item.first));
    w.push_back(static_cast<uint32_t>(item.first >> 32));
    w.push_back(static_cast<uint32_t>(item.second.size()));
    w.insert(w.end(), item.second.begin(), item.second.end());
  }
  return w;
}

// `gathered` = concatenation of every rank's frame (all the same length as `local`). Returns -1 when all
// ranks agree, else the first rank that differs. Malformed input throws.
static int validate_gathered(const std::vector<uint32_t>& local, const std::vector<uint32_t>& gathered, int participants) {
  if (participants <= 0) throw std::invalid_argument("consensus topology has no participants");
  if (gathered.size() != local.size() * static_cast<size_t>(participants))
    throw std::runtime_error("consensus returned " + std::to_string(gathered.size()) + " words; expected " +
                             std::to_string(local.size() * participants) + " for " + std::to_string(participants) + " ranks");
  for (int r = 0; r < participants; ++r)
    if (!std::equal(local.begin(), local.end(), gathered.begin() + static_cast<size_t>(r) * local.size())) return r;
  return -1;
}

// observations per rank: 0 incomplete, 1 complete, 2 failed. One entry per work item, rank-major.
// Resolution: 0 Incomplete, 1 Complete, 2 FailedPending (a rank failed, another still runs), 3 FailedComplete.
static std::vector<int> resolve_completions(const std::vector<uint32_t>& gathered, int participants, int items) {
  if (static_cast<int>(gathered.size()) != participants * items) throw std::runtime_error("malformed completion gather");
  std::vector<int> out(items, 0);
  for (int i = 0; i < items; ++i) {
    bool any_failed = false, any_incomplete = false;
    for (int r = 0; r < participants; ++r) {
      const uint32_t v = gathered[static_cast<size_t>(r) * items + i];
      if (v > 2) throw std::runtime_error("invalid completion status at rank " + std::to_string(r));
      any_failed |= v == 2;
      any_incomplete |= v == 0;
    }
    out[i] = any_failed ? (any_incomplete ? 2 : 3) : (any_incomplete ? 0 : 1);
  }
  return out;
}

void bind_runtime(py::module_& m) {
  m.def("balanced_contiguous_range", &balanced_range);
  m.def("aligned_partition_units", &aligned_partition_units);
  py::class_<BlockManager>(m, "BlockManager")
      .def(py::init<int64_t, const std::string&>(), py::arg("num_pages"), py::arg("eviction") = "lru")
      .def("free_pages", &BlockManager::free_pages)
      .def("cached_pages", &BlockManager::cached_pages)
      .def_property_readonly("num_pages", &BlockManager::num_pages)
      .def_readonly("evictions", &BlockManager::evictions_)
      .def("alloc", &BlockManager::alloc)
      .def("retain", &BlockManager::retain)
      .def("release", &BlockManager::release)
      .def("seal", &BlockManager::seal)
      .def("match_prefix", &BlockManager::match_prefix)
      .def("seal_prefix", &BlockManager::seal_prefix)
      .def("refcount", &BlockManager::refcount)
      .def("lookup", &BlockManager::lookup)
      .def("take_evicted", &BlockManager::take_evicted)
      .def_static("chain_hash", &BlockManager::chain_hash);
  py::class_<WorkItem>(m, "WorkItem")
      .def_readonly("work_id", &WorkItem::work_id)
      .def_readonly("request_id", &WorkItem::request_id)
      .def_readonly("kind", &WorkItem::kind)
      .def_readonly("tokens", &WorkItem::tokens);
  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<int64_t, int64_t, int64_t, int64_t>(), py::arg("max_batch") = 32, py::arg("max_step_tokens") = 8192,
           py::arg("max_waiting") = 1024, py::arg("prefill_chunk") = 2048)
      .def("submit", &Scheduler::submit, py::arg("prompt_tokens"), py::arg("max_new_tokens"), py::arg("deadline") = 0.0)
      .def("cancel", &Scheduler::cancel)
      .def("plan_step", &Scheduler::plan_step, py::arg("now") = 0.0)
      .def("complete", &Scheduler::complete, py::arg("work_id"), py::arg("tokens"), py::arg("generated"),
           py::arg("stop") = false, py::arg("failed") = false)
      .def("poison", &Scheduler::poison)
      .def_property_readonly("poisoned", &Scheduler::poisoned)
      .def("request", &Scheduler::request)
      .def("report", &Scheduler::report)
      .def("reap", &Scheduler::reap);
  m.def("encode_schedule", &encode_schedule);
  m.def("validate_gathered", &validate_gathered);
  m.def("resolve_completions", &resolve_completions);
}

}  // namespace eredu
