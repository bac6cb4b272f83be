// Exactly-once work accounting for asynchronous producer / consumer training.
//
// Every Target output is one record that moves through
//   produced -> dispatched(expected consumers) -> released | completed | failed
//   released -> committed(optimizer step)          produced -> discard_pending -> discarded
//   released -> discarded (cooperative shutdown)   anything live -> discarded after an owner fence
// Residency (outputs, bytes, peaks) is tracked and must return to zero; a commit rejects repeated
// steps, a wrong number of unique items, wrong multiplicity and items that are not released.
// (Behavioural counterpart of aspec/work_lifecycle.py:86-434 in the reference.)
#include <algorithm>
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

namespace {

enum State { Produced, Dispatched, Released, Completed, Failed, Committed, DiscardPending, Discarded };
const char* kStateNames[] = {"produced", "dispatched", "released", "completed", "failed", "committed",
                             "discard_pending", "discarded"};

struct Record {
  std::string execution_id, work_id, work_kind, data_id, key;
  long long size_bytes = 0;
  State state = Produced;
  int expected_consumers = 0;
  std::map<std::string, std::string> outcomes;  // participant -> outcome
  std::string release_outcome;
  long long optimizer_step = -1;
  bool resident = true;
};

struct Ledger {
  std::mutex mu;
  std::map<std::string, Record> records;
  std::map<std::string, std::string> key_to_execution;
  std::map<long long, std::vector<std::string>> commits;
  std::vector<std::string> errors;
  long long resident_outputs = 0, resident_bytes = 0, peak_outputs = 0, peak_bytes = 0;
  std::string last_error, scratch;

  int fail(const std::string& msg) {
    errors.push_back(msg);
    last_error = msg;
    return 1;
  }
  void drop(Record& r) {
    if (!r.resident) return;
    r.resident = false;
    resident_outputs -= 1;
    resident_bytes -= r.size_bytes;
    key_to_execution.erase(r.key);
  }
};

std::vector<std::string> split_lines(const char* s) {
  std::vector<std::string> out;
  std::string cur;
  for (const char* p = s; *p; ++p) {
    if (*p == '\n') { out.push_back(cur); cur.clear(); } else cur.push_back(*p);
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o.push_back('\\'); o.push_back(c); }
    else if (c == '\n') o += "\\n";
    else o.push_back(c);
  }
  return o;
}

}  // namespace

extern "C" {

void* ab_ledger_create() { return new Ledger(); }
void ab_ledger_destroy(void* h) { delete static_cast<Ledger*>(h); }
const char* ab_ledger_last_error(void* h) { return static_cast<Ledger*>(h)->last_error.c_str(); }

// Batch registration: n outputs; the whole batch is validated before anything is recorded.
// Arrays of C strings: execution_id, work_id, work_kind, data_id, key; sizes in bytes.
int ab_ledger_register(void* h, int n, const char** execution_ids, const char** work_ids, const char** kinds,
                       const char** data_ids, const char** keys, const long long* sizes) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  std::set<std::string> seen_exec, seen_key;
  for (int i = 0; i < n; ++i) {
    if (L->records.count(execution_ids[i]) || !seen_exec.insert(execution_ids[i]).second)
      return L->fail(std::string("duplicate execution_id: ") + execution_ids[i]);
    if (L->key_to_execution.count(keys[i]) || !seen_key.insert(keys[i]).second)
      return L->fail(std::string("duplicate live feature key: ") + keys[i]);
    if (sizes[i] < 0) return L->fail(std::string("negative output size for ") + execution_ids[i]);
  }
  for (int i = 0; i < n; ++i) {
    Record r;
    r.execution_id = execution_ids[i];
    r.work_id = work_ids[i];
    r.work_kind = kinds[i];
    r.data_id = data_ids[i];
    r.key = keys[i];
    r.size_bytes = sizes[i];
    L->key_to_execution[r.key] = r.execution_id;
    L->records[r.execution_id] = r;
    L->resident_outputs += 1;
    L->resident_bytes += sizes[i];
  }
  L->peak_outputs = std::max(L->peak_outputs, L->resident_outputs);
  L->peak_bytes = std::max(L->peak_bytes, L->resident_bytes);
  return 0;
}

int ab_ledger_mark_dispatched(void* h, const char* execution_id, int expected_consumers) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  auto it = L->records.find(execution_id);
  if (it == L->records.end()) return L->fail(std::string("dispatch references unknown execution_id: ") + execution_id);
  Record& r = it->second;
  if (r.state != Produced)
    return L->fail(std::string("cannot dispatch ") + execution_id + " from state '" + kStateNames[r.state] + "'");
  if (expected_consumers <= 0) return L->fail(std::string("expected_consumers must be positive for ") + execution_id);
  r.state = Dispatched;
  r.expected_consumers = expected_consumers;
  return 0;
}

int ab_ledger_release(void* h, const char* execution_id, const char* data_id, const char* key,
                      const char* participant, const char* outcome) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  auto it = L->records.find(execution_id);
  if (it == L->records.end()) return L->fail(std::string("release references unknown execution_id: ") + execution_id);
  Record& r = it->second;
  if (r.data_id != data_id || r.key != key) return L->fail(std::string("release identity mismatch for ") + execution_id);
  if (r.state != Dispatched)
    return L->fail(std::string("cannot release ") + execution_id + " from state '" + kStateNames[r.state] + "'");
  if (r.outcomes.count(participant))
    return L->fail(std::string("duplicate release of ") + execution_id + " by " + participant);
  const std::string oc = outcome;
  if (oc != "consumed" && oc != "discarded_after_error")
    return L->fail(std::string("invalid release outcome for ") + execution_id + ": " + oc);
  r.outcomes[participant] = oc;
  if ((int)r.outcomes.size() > r.expected_consumers) return L->fail(std::string("too many releases for ") + execution_id);
  if ((int)r.outcomes.size() < r.expected_consumers) return 0;
  bool failed = false;
  for (auto& kv : r.outcomes) failed |= kv.second == "discarded_after_error";
  if (failed) { r.release_outcome = "discarded_after_error"; r.state = Failed; }
  else if (r.work_kind == "train") { r.release_outcome = "consumed"; r.state = Released; }
  else { r.release_outcome = "consumed"; r.state = Completed; }
  L->drop(r);
  return 0;
}

int ab_ledger_begin_discard(void* h, const char* execution_id) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  auto it = L->records.find(execution_id);
  if (it == L->records.end()) return L->fail(std::string("discard references unknown execution_id: ") + execution_id);
  if (it->second.state != Produced)
    return L->fail(std::string("cannot discard ") + execution_id + " from state '" + kStateNames[it->second.state] + "'");
  it->second.state = DiscardPending;
  return 0;
}

int ab_ledger_confirm_discarded(void* h, const char* execution_id) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  auto it = L->records.find(execution_id);
  if (it == L->records.end())
    return L->fail(std::string("discard confirmation references unknown execution_id: ") + execution_id);
  if (it->second.state != DiscardPending)
    return L->fail(std::string("cannot confirm discard of ") + execution_id + " from state '" +
                   kStateNames[it->second.state] + "'");
  it->second.state = Discarded;
  it->second.release_outcome = "unused_output_discarded";
  L->drop(it->second);
  return 0;
}

// execution_ids: '\n'-separated, may repeat (one entry per consumer report).
int ab_ledger_commit(void* h, long long optimizer_step, const char* execution_ids, int expected_unique,
                     int expected_occurrences) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  if (L->commits.count(optimizer_step)) return L->fail("optimizer step already committed: " + std::to_string(optimizer_step));
  std::map<std::string, int> counts;
  for (auto& id : split_lines(execution_ids)) counts[id] += 1;
  if ((int)counts.size() != expected_unique)
    return L->fail("optimizer step " + std::to_string(optimizer_step) + " has " + std::to_string(counts.size()) +
                   " unique work items; expected " + std::to_string(expected_unique));
  for (auto& kv : counts)
    if (kv.second != expected_occurrences)
      return L->fail("optimizer step " + std::to_string(optimizer_step) + " has invalid work multiplicity: " + kv.first);
  for (auto& kv : counts) {
    auto it = L->records.find(kv.first);
    if (it == L->records.end())
      return L->fail("optimizer step " + std::to_string(optimizer_step) + " references unknown work: " + kv.first);
    if (it->second.state != Released)
      return L->fail("optimizer step " + std::to_string(optimizer_step) + " cannot commit " + kv.first + " from state '" +
                     kStateNames[it->second.state] + "'");
  }
  std::vector<std::string> ids;
  for (auto& kv : counts) {
    Record& r = L->records[kv.first];
    r.state = Committed;
    r.optimizer_step = optimizer_step;
    ids.push_back(kv.first);
  }
  L->commits[optimizer_step] = ids;
  return 0;
}

// mode 0: released-but-uncommitted -> discarded (cooperative shutdown)
// mode 1: the listed execution ids, any live state, after an owner fence
// mode 2: every live record, after an owner fence
int ab_ledger_discard(void* h, int mode, const char* execution_ids) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  int n = 0;
  auto live = [](State s) { return s == Produced || s == Dispatched || s == DiscardPending || s == Released; };
  if (mode == 0) {
    for (auto& kv : L->records)
      if (kv.second.state == Released) {
        kv.second.state = Discarded;
        kv.second.release_outcome = "released_uncommitted_discarded";
        ++n;
      }
  } else if (mode == 1) {
    for (auto& id : split_lines(execution_ids)) {
      auto it = L->records.find(id);
      if (it == L->records.end()) { L->fail("owner-fence discard references unknown execution_id: " + id); return -1; }
      if (!live(it->second.state)) continue;
      it->second.state = Discarded;
      it->second.release_outcome = "discarded_after_owner_fence";
      L->drop(it->second);
      ++n;
    }
  } else {
    for (auto& kv : L->records)
      if (live(kv.second.state)) {
        kv.second.state = Discarded;
        kv.second.release_outcome = "discarded_after_owner_fence";
        L->drop(kv.second);
        ++n;
      }
  }
  return n;
}

long long ab_ledger_resident_outputs(void* h) { return static_cast<Ledger*>(h)->resident_outputs; }
long long ab_ledger_resident_bytes(void* h) { return static_cast<Ledger*>(h)->resident_bytes; }

// JSON document with counters, per-state counts, committed work ids and the validation verdict.
const char* ab_ledger_status(void* h) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  std::map<std::string, long long> per_state;
  std::set<std::string> committed_work;
  bool unique_commits = true;
  long long incomplete = 0;
  for (auto& kv : L->records) {
    per_state[kStateNames[kv.second.state]] += 1;
    if (kv.second.state == Committed && !committed_work.insert(kv.second.work_id).second) unique_commits = false;
    if (kv.second.state == Produced || kv.second.state == Dispatched || kv.second.state == DiscardPending ||
        kv.second.state == Released)
      incomplete += 1;
  }
  bool contiguous = true;
  long long prev = 0;
  bool first = true;
  for (auto& kv : L->commits) {
    if (!first && kv.first != prev + 1) contiguous = false;
    prev = kv.first;
    first = false;
  }
  const bool validated = L->errors.empty() && L->resident_outputs == 0 && L->resident_bytes == 0 && incomplete == 0 &&
                         contiguous && unique_commits;
  std::string o;
  auto num = [&](long long v) { o += std::to_string(v); };
  o += "{\"records\":"; num((long long)L->records.size());
  o += ",\"states\":{";
  bool c = false;
  for (auto& kv : per_state) { o += (c ? "," : ""); o += "\"" + kv.first + "\":"; num(kv.second); c = true; }
  o += "},\"resident_outputs\":"; num(L->resident_outputs);
  o += ",\"resident_bytes\":"; num(L->resident_bytes);
  o += ",\"peak_resident_outputs\":"; num(L->peak_outputs);
  o += ",\"peak_resident_bytes\":"; num(L->peak_bytes);
  o += ",\"committed_steps\":[";
  c = false;
  for (auto& kv : L->commits) { o += (c ? "," : ""); num(kv.first); c = true; }
  o += "],\"committed_work_ids\":[";
  c = false;
  for (auto& w : committed_work) { o += (c ? "," : ""); o += "\"" + json_escape(w) + "\""; c = true; }
  o += "],\"incomplete\":"; num(incomplete);
  o += std::string(",\"contiguous_steps\":") + (contiguous ? "true" : "false");
  o += std::string(",\"unique_committed_work\":") + (unique_commits ? "true" : "false");
  o += ",\"errors\":[";
  c = false;
  for (auto& e : L->errors) { o += (c ? "," : ""); o += "\"" + json_escape(e) + "\""; c = true; }
  o += std::string("],\"validated\":") + (validated ? "true" : "false") + "}";
  L->scratch = o;
  return L->scratch.c_str();
}

const char* ab_ledger_state_of(void* h, const char* execution_id) {
  Ledger* L = static_cast<Ledger*>(h);
  std::lock_guard<std::mutex> g(L->mu);
  auto it = L->records.find(execution_id);
  return it == L->records.end() ? "" : kStateNames[it->second.state];
}

}  // extern "C"
