// Residency accounting of the host runtime: which copy of which weight / cache unit lives in which memory tier, under
// byte budgets, with reserve -> publish / rollback transactions, pins, eviction order and transfer generations; and the
// process-wide byte pool that KV-cache tiers reserve from.
//
// Behavioural counterpart of eredu-core/src/residency.rs (`ResidencyLedger`: reserve_copy :1328, publish_reserved :1452,
// rollback_reserved :1507, next_transfer_generation / resolve_transfer :1525-1570, pin / unpin / touch / evict
// :1571-1680, telemetry :801-940) and eredu-core/src/cache.rs:48-450 (device / host / transfer / disk reservations).
// The ledger knows nothing about tensors: callers move the bytes and tell it what happened.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace eredu {

namespace {

constexpr int kTiers = 3;  // 0 device, 1 host, 2 disk
const char* kTierName[kTiers] = {"device", "host", "disk"};

int tier_index(const std::string& t) {
  for (int i = 0; i < kTiers; ++i)
    if (t == kTierName[i]) return i;
  throw std::invalid_argument("unknown memory tier '" + t + "' (device | host | disk)");
}

enum class Policy { Pinned, Windowed, Cacheable };

Policy parse_policy(const std::string& p) {
  if (p == "pinned") return Policy::Pinned;
  if (p == "windowed") return Policy::Windowed;
  if (p == "cacheable") return Policy::Cacheable;
  throw std::invalid_argument("unknown residency policy '" + p + "' (pinned | windowed | cacheable)");
}

struct Copy {
  bool resident = false;
  bool reserved = false;   // bytes are charged, contents not yet valid
  int pins = 0;
  uint64_t last_use = 0;
  uint64_t uses = 0;
  uint64_t generation = 0;  // newest transfer issued for this copy
};

struct Unit {
  std::string id;
  int64_t bytes = 0;
  Policy policy = Policy::Cacheable;
  int home = 2;
  Copy copy[kTiers];
};

}  // namespace

class ResidencyLedger {
 public:
  ResidencyLedger(int64_t device_budget, int64_t host_budget, int64_t disk_budget, const std::string& eviction) {
    budget_[0] = device_budget;
    budget_[1] = host_budget;
    budget_[2] = disk_budget;
    if (eviction != "lru" && eviction != "lfu") throw std::invalid_argument("eviction must be lru or lfu");
    lfu_ = eviction == "lfu";
  }

  void add_unit(const std::string& id, int64_t bytes, const std::string& policy, const std::string& home) {
    if (id.empty()) throw std::invalid_argument("unit id must not be empty");
    if (bytes < 0) throw std::invalid_argument("unit size must not be negative");
    if (units_.count(id)) throw std::invalid_argument("duplicate unit '" + id + "'");
    Unit u;
    u.id = id;
    u.bytes = bytes;
    u.policy = parse_policy(policy);
    u.home = tier_index(home);
    u.copy[u.home].resident = true;  // the home copy exists from the start and is never evicted
    used_[u.home] += bytes;
    units_[id] = u;
  }

  // Charges the unit's bytes to the tier, evicting unpinned cacheable / windowed copies in policy order when the budget
  // needs it. Returns the ids whose copies were dropped (the caller frees their memory). Throws when the bytes cannot
  // be found; nothing changes in that case.
  std::vector<std::string> reserve(const std::string& id, const std::string& tier) {
    Unit& u = unit(id);
    const int t = tier_index(tier);
    Copy& c = u.copy[t];
    if (c.resident || c.reserved) throw std::runtime_error("unit '" + id + "' already has a copy in " + tier);
    std::vector<std::string> victims;
    if (budget_[t] >= 0) {
      int64_t need = used_[t] + u.bytes - budget_[t];
      if (need > 0) {
        std::vector<Unit*> cands;
        for (auto& kv : units_) {
          Unit& o = kv.second;
          const Copy& oc = o.copy[t];
          if (&o == &u || !oc.resident || oc.pins > 0 || o.home == t || o.policy == Policy::Pinned) continue;
          cands.push_back(&o);
        }
        std::sort(cands.begin(), cands.end(), [&](const Unit* a, const Unit* b) {
          const Copy &x = a->copy[t], &y = b->copy[t];
          if (lfu_ && x.uses != y.uses) return x.uses < y.uses;
          if (x.last_use != y.last_use) return x.last_use < y.last_use;
          return a->id < b->id;
        });
        int64_t freed = 0;
        size_t n = 0;
        while (n < cands.size() && freed < need) freed += cands[n++]->bytes;
        if (freed < need) {
          ++refused_[t];
          throw std::runtime_error("tier " + tier + " cannot hold unit '" + id + "': " + std::to_string(need - freed) +
                                   " bytes short after evicting everything evictable");
        }
        for (size_t i = 0; i < n; ++i) {
          drop(*cands[i], t);
          victims.push_back(cands[i]->id);
        }
      }
    }
    c.reserved = true;
    used_[t] += u.bytes;
    return victims;
  }

  void publish(const std::string& id, const std::string& tier) {
    Copy& c = unit(id).copy[tier_index(tier)];
    if (!c.reserved) throw std::runtime_error("publish without a reservation for '" + id + "' in " + tier);
    c.reserved = false;
    c.resident = true;
    c.last_use = ++clock_;
    c.uses = 0;
  }

  void rollback(const std::string& id, const std::string& tier) {
    Unit& u = unit(id);
    const int t = tier_index(tier);
    if (!u.copy[t].reserved) throw std::runtime_error("rollback without a reservation for '" + id + "' in " + tier);
    u.copy[t].reserved = false;
    used_[t] -= u.bytes;
  }

  // A transfer is identified by the generation handed out when it was issued; a completion carrying an older
  // generation than the copy's newest one is stale (the copy was evicted and re-requested meanwhile) and is ignored.
  uint64_t begin_transfer(const std::string& id, const std::string& tier) {
    Copy& c = unit(id).copy[tier_index(tier)];
    c.generation = ++generation_;
    return c.generation;
  }

  bool resolve_transfer(const std::string& id, const std::string& tier, uint64_t generation, const std::string& from,
                        double seconds) {
    Unit& u = unit(id);
    const int t = tier_index(tier);
    Copy& c = u.copy[t];
    if (c.generation != generation || !c.reserved) {
      ++stale_transfers_;
      return false;
    }
    publish(id, tier);
    const int f = tier_index(from);
    transfer_bytes_[f][t] += u.bytes;
    transfer_count_[f][t] += 1;
    transfer_seconds_[f][t] += seconds;
    return true;
  }

  void pin(const std::string& id, const std::string& tier) {
    Copy& c = unit(id).copy[tier_index(tier)];
    if (!c.resident) throw std::runtime_error("cannot pin '" + id + "': no resident copy in " + tier);
    ++c.pins;
  }

  void unpin(const std::string& id, const std::string& tier) {
    Copy& c = unit(id).copy[tier_index(tier)];
    if (c.pins > 0) --c.pins;
  }

  void touch(const std::string& id, const std::string& tier) {
    Copy& c = unit(id).copy[tier_index(tier)];
    if (!c.resident) throw std::runtime_error("cannot touch '" + id + "': no resident copy in " + tier);
    c.last_use = ++clock_;
    ++c.uses;
  }

  bool evict(const std::string& id, const std::string& tier) {
    Unit& u = unit(id);
    const int t = tier_index(tier);
    const Copy& c = u.copy[t];
    if (!c.resident) return false;
    if (c.pins > 0) throw std::runtime_error("cannot evict pinned copy of '" + id + "' in " + tier);
    if (u.home == t) throw std::runtime_error("cannot evict the home copy of '" + id + "'");
    drop(u, t);
    return true;
  }

  bool is_resident(const std::string& id, const std::string& tier) { return unit(id).copy[tier_index(tier)].resident; }
  int64_t resident_bytes(const std::string& tier) const { return used_[tier_index(tier)]; }

  void record_prefetch(const std::string& tier, const std::string& outcome) {
    const int t = tier_index(tier);
    if (outcome == "hit") ++prefetch_hit_[t];
    else if (outcome == "late") ++prefetch_late_[t];
    else if (outcome == "miss") ++prefetch_miss_[t];
    else throw std::invalid_argument("prefetch outcome must be hit, late or miss");
  }

  void record_stall(double seconds) {
    ++stalls_;
    stall_seconds_ += seconds;
  }

  py::dict report() const {
    py::dict d;
    for (int t = 0; t < kTiers; ++t) {
      py::dict tier;
      int64_t units = 0;
      for (const auto& kv : units_) units += kv.second.copy[t].resident ? 1 : 0;
      tier["budget_bytes"] = budget_[t] < 0 ? py::object(py::none()) : py::object(py::int_(budget_[t]));
      tier["resident_bytes"] = used_[t];
      tier["resident_units"] = units;
      tier["evictions"] = evictions_[t];
      tier["evicted_bytes"] = evicted_bytes_[t];
      tier["refused"] = refused_[t];
      tier["prefetch"] = py::dict(py::arg("hit") = prefetch_hit_[t], py::arg("late") = prefetch_late_[t],
                                  py::arg("miss") = prefetch_miss_[t]);
      d[kTierName[t]] = tier;
    }
    py::dict transfers;
    for (int f = 0; f < kTiers; ++f)
      for (int t = 0; t < kTiers; ++t)
        if (transfer_count_[f][t] > 0)
          transfers[(std::string(kTierName[f]) + "_to_" + kTierName[t]).c_str()] =
              py::dict(py::arg("count") = transfer_count_[f][t], py::arg("bytes") = transfer_bytes_[f][t],
                       py::arg("seconds") = transfer_seconds_[f][t]);
    d["transfers"] = transfers;
    d["stale_transfers"] = stale_transfers_;
    d["stalls"] = stalls_;
    d["stall_seconds"] = stall_seconds_;
    d["units"] = static_cast<int64_t>(units_.size());
    return d;
  }

 private:
  Unit& unit(const std::string& id) {
    auto it = units_.find(id);
    if (it == units_.end()) throw std::out_of_range("unknown unit '" + id + "'");
    return it->second;
  }

  void drop(Unit& u, int t) {
    u.copy[t].resident = false;
    u.copy[t].uses = 0;
    used_[t] -= u.bytes;
    ++evictions_[t];
    evicted_bytes_[t] += u.bytes;
  }

  std::map<std::string, Unit> units_;
  int64_t budget_[kTiers];
  int64_t used_[kTiers] = {0, 0, 0};
  bool lfu_ = false;
  uint64_t clock_ = 0, generation_ = 0;
  int64_t evictions_[kTiers] = {0, 0, 0}, evicted_bytes_[kTiers] = {0, 0, 0}, refused_[kTiers] = {0, 0, 0};
  int64_t prefetch_hit_[kTiers] = {0, 0, 0}, prefetch_late_[kTiers] = {0, 0, 0}, prefetch_miss_[kTiers] = {0, 0, 0};
  int64_t transfer_bytes_[kTiers][kTiers] = {}, transfer_count_[kTiers][kTiers] = {};
  double transfer_seconds_[kTiers][kTiers] = {};
  int64_t stale_transfers_ = 0, stalls_ = 0;
  double stall_seconds_ = 0.0;
};

// Process-wide byte pool shared by every cache of the process: a reservation either fits the kind's budget or is
// refused; releasing returns the bytes. Kinds: device, host, transfer (staging in flight), disk.
class CachePool {
 public:
  CachePool(int64_t device, int64_t host, int64_t transfer, int64_t disk) {
    budget_["device"] = device;
    budget_["host"] = host;
    budget_["transfer"] = transfer;
    budget_["disk"] = disk;
    for (auto& kv : budget_) used_[kv.first] = 0;
  }

  int64_t reserve(const std::string& kind, int64_t bytes) {
    auto it = budget_.find(kind);
    if (it == budget_.end()) throw std::invalid_argument("unknown pool kind '" + kind + "'");
    if (bytes < 0) throw std::invalid_argument("reservation size must not be negative");
    if (it->second >= 0 && used_[kind] + bytes > it->second) {
      ++refused_;
      return -1;
    }
    used_[kind] += bytes;
    peak_[kind] = std::max(peak_[kind], used_[kind]);
    const int64_t handle = ++next_;
    live_[handle] = {kind, bytes};
    return handle;
  }

  void release(int64_t handle) {
    auto it = live_.find(handle);
    if (it == live_.end()) throw std::out_of_range("unknown or already released reservation");
    used_[it->second.first] -= it->second.second;
    live_.erase(it);
  }

  int64_t used(const std::string& kind) const {
    auto it = used_.find(kind);
    if (it == used_.end()) throw std::invalid_argument("unknown pool kind '" + kind + "'");
    return it->second;
  }

  py::dict report() const {
    py::dict d;
    for (const auto& kv : budget_) {
      auto p = peak_.find(kv.first);
      d[kv.first.c_str()] = py::dict(py::arg("budget_bytes") = kv.second < 0 ? py::object(py::none()) : py::object(py::int_(kv.second)),
                                     py::arg("used_bytes") = used_.at(kv.first),
                                     py::arg("peak_bytes") = p == peak_.end() ? int64_t(0) : p->second);
    }
    d["live_reservations"] = static_cast<int64_t>(live_.size());
    d["refused"] = refused_;
    return d;
  }

 private:
  std::map<std::string, int64_t> budget_, used_, peak_;
  std::map<int64_t, std::pair<std::string, int64_t>> live_;
  int64_t next_ = 0, refused_ = 0;
};

void bind_residency(py::module_& m) {
  py::class_<ResidencyLedger>(m, "ResidencyLedger")
      .def(py::init<int64_t, int64_t, int64_t, const std::string&>(), py::arg("device_budget_bytes") = -1,
           py::arg("host_budget_bytes") = -1, py::arg("disk_budget_bytes") = -1, py::arg("eviction") = "lru")
      .def("add_unit", &ResidencyLedger::add_unit, py::arg("id"), py::arg("bytes"), py::arg("policy") = "cacheable",
           py::arg("home") = "disk")
      .def("reserve", &ResidencyLedger::reserve)
      .def("publish", &ResidencyLedger::publish)
      .def("rollback", &ResidencyLedger::rollback)
      .def("begin_transfer", &ResidencyLedger::begin_transfer)
      .def("resolve_transfer", &ResidencyLedger::resolve_transfer, py::arg("id"), py::arg("tier"), py::arg("generation"),
           py::arg("source"), py::arg("seconds") = 0.0)
      .def("pin", &ResidencyLedger::pin)
      .def("unpin", &ResidencyLedger::unpin)
      .def("touch", &ResidencyLedger::touch)
      .def("evict", &ResidencyLedger::evict)
      .def("is_resident", &ResidencyLedger::is_resident)
      .def("resident_bytes", &ResidencyLedger::resident_bytes)
      .def("record_prefetch", &ResidencyLedger::record_prefetch)
      .def("record_stall", &ResidencyLedger::record_stall)
      .def("report", &ResidencyLedger::report);
  py::class_<CachePool>(m, "CachePool")
      .def(py::init<int64_t, int64_t, int64_t, int64_t>(), py::arg("device_bytes") = -1, py::arg("host_bytes") = -1,
           py::arg("transfer_bytes") = -1, py::arg("disk_bytes") = -1)
      .def("reserve", &CachePool::reserve)
      .def("release", &CachePool::release)
      .def("used", &CachePool::used)
      .def("report", &CachePool::report);
}

}  // namespace eredu
