// Fixed-size ring of transfer slots with generation-checked leases and a frozen reader audience.
//
// Semantics (the reference keeps the same state machine in Python,
// aspec/transfer/mooncake/p2p.py:315-465):
//   * acquire(owner, timeout) takes the first free slot, bumps its generation and returns the
//     lease (slot, generation, owner); it blocks on a condition variable up to the deadline;
//   * release must name the live lease exactly, otherwise it is "stale or duplicate";
//   * register_readers freezes the set of readers before any descriptor becomes visible; each
//     reader acknowledges once, the last acknowledgement frees the slot; a slot with readers
//     pending cannot be released directly;
//   * release_acknowledged is idempotent over a bounded history (max(64, 32 * slots) leases), so
//     a lost acknowledgement can be retried without freeing a newer generation.
// The generation doubles as the value of the device-side flag word a consumer kernel waits for.
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <set>
#include <string>
#include <vector>

namespace {

struct Lease {
  int slot = -1;
  long long generation = 0;
  std::string owner;
  bool operator<(const Lease& o) const {
    if (slot != o.slot) return slot < o.slot;
    if (generation != o.generation) return generation < o.generation;
    return owner < o.owner;
  }
  bool operator==(const Lease& o) const { return slot == o.slot && generation == o.generation && owner == o.owner; }
};

struct Slot {
  long long generation = 0;
  bool live = false;
  std::string owner;
  bool readers_registered = false;
  std::set<std::string> audience, pending;
};

struct Ring {
  std::mutex mu;
  std::condition_variable cv;
  std::vector<Slot> slots;
  std::deque<Lease> history;
  std::set<Lease> history_set;
  size_t history_limit;
  explicit Ring(int n) : slots(n), history_limit(std::max<size_t>(64, size_t(n) * 32)) {}

  void remember(const Lease& l) {
    history.push_back(l);
    history_set.insert(l);
    while (history.size() > history_limit) {
      history_set.erase(history.front());
      history.pop_front();
    }
  }
  void free_slot(Slot& s, int index) {
    remember(Lease{index, s.generation, s.owner});
    s.live = false;
    s.owner.clear();
    s.readers_registered = false;
    s.audience.clear();
    s.pending.clear();
    cv.notify_all();
  }
};

enum : int {
  kOk = 0, kTimeout = 1, kStale = 2, kReadersPending = 3, kAlreadyRegistered = 4, kNotAReader = 5,
  kBadArgument = 6, kAlreadyAcknowledged = 7,
};

}  // namespace

extern "C" {

void* ab_ring_create(int slots) { return slots >= 1 ? new Ring(slots) : nullptr; }
void ab_ring_destroy(void* h) { delete static_cast<Ring*>(h); }
int ab_ring_slots(void* h) { return (int)static_cast<Ring*>(h)->slots.size(); }

int ab_ring_in_use(void* h) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  int n = 0;
  for (auto& s : r->slots) n += s.live;
  return n;
}

// timeout_s < 0: wait forever.  Writes slot and generation.
int ab_ring_acquire(void* h, const char* owner, double timeout_s, int* slot, long long* generation) {
  Ring* r = static_cast<Ring*>(h);
  std::unique_lock<std::mutex> lk(r->mu);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s < 0 ? 0 : timeout_s);
  for (;;) {
    for (size_t i = 0; i < r->slots.size(); ++i) {
      Slot& s = r->slots[i];
      if (!s.live) {
        s.live = true;
        s.generation += 1;
        s.owner = owner;
        *slot = (int)i;
        *generation = s.generation;
        return kOk;
      }
    }
    if (timeout_s < 0) {
      r->cv.wait(lk);
    } else if (r->cv.wait_until(lk, deadline) == std::cv_status::timeout) {
      bool any_free = false;
      for (auto& s : r->slots) any_free |= !s.live;
      if (!any_free) return kTimeout;
    }
  }
}

int ab_ring_release(void* h, int slot, long long generation, const char* owner) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (slot < 0 || slot >= (int)r->slots.size()) return kBadArgument;
  Slot& s = r->slots[slot];
  if (!s.live || s.generation != generation || s.owner != owner) return kStale;
  if (!s.pending.empty()) return kReadersPending;
  r->free_slot(s, slot);
  return kOk;
}

// readers: '\n'-separated names.  Freezes the audience; may be called once per lease.
int ab_ring_register_readers(void* h, int slot, long long generation, const char* owner, const char* readers) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (slot < 0 || slot >= (int)r->slots.size()) return kBadArgument;
  Slot& s = r->slots[slot];
  if (!s.live || s.generation != generation || s.owner != owner) return kStale;
  if (s.readers_registered) return kAlreadyRegistered;
  std::set<std::string> names;
  const char* p = readers;
  while (*p) {
    const char* e = strchr(p, '\n');
    std::string name = e ? std::string(p, e) : std::string(p);
    if (!name.empty()) names.insert(name);
    if (!e) break;
    p = e + 1;
  }
  if (names.empty()) return kBadArgument;
  s.audience = names;
  s.pending = names;
  s.readers_registered = true;
  return kOk;
}

int ab_ring_reader_pending(void* h, int slot, long long generation, const char* owner, const char* reader) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (slot < 0 || slot >= (int)r->slots.size()) return 0;
  Slot& s = r->slots[slot];
  if (!s.live || s.generation != generation || s.owner != owner) return 0;
  return s.pending.count(reader) ? 1 : 0;
}

// One reader acknowledges.  *freed is set when this was the last one and the slot became free.
int ab_ring_release_reader(void* h, int slot, long long generation, const char* owner, const char* reader, int* freed) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  *freed = 0;
  if (slot < 0 || slot >= (int)r->slots.size()) return kBadArgument;
  Slot& s = r->slots[slot];
  if (!s.live || s.generation != generation || s.owner != owner) {
    return r->history_set.count(Lease{slot, generation, owner}) ? kAlreadyAcknowledged : kStale;
  }
  if (!s.audience.count(reader)) return kNotAReader;
  if (!s.pending.erase(reader)) return kAlreadyAcknowledged;
  if (s.pending.empty()) {
    r->free_slot(s, slot);
    *freed = 1;
  }
  return kOk;
}

// Idempotent release used by acknowledgement retries: freeing a lease already in the bounded
// history is a success; a lease that is neither live nor remembered is stale.
int ab_ring_release_acknowledged(void* h, int slot, long long generation, const char* owner) {
  Ring* r = static_cast<Ring*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (slot < 0 || slot >= (int)r->slots.size()) return kBadArgument;
  Slot& s = r->slots[slot];
  if (s.live && s.generation == generation && s.owner == owner) {
    if (!s.pending.empty()) return kReadersPending;
    r->free_slot(s, slot);
    return kOk;
  }
  return r->history_set.count(Lease{slot, generation, owner}) ? kAlreadyAcknowledged : kStale;
}

int ab_ring_wait_until_empty(void* h, double timeout_s) {
  Ring* r = static_cast<Ring*>(h);
  std::unique_lock<std::mutex> lk(r->mu);
  auto empty = [&] { for (auto& s : r->slots) if (s.live) return false; return true; };
  if (timeout_s < 0) { r->cv.wait(lk, empty); return 1; }
  return r->cv.wait_for(lk, std::chrono::duration<double>(timeout_s), empty) ? 1 : 0;
}

}  // extern "C"
