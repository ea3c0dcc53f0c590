// Paged cache bookkeeping on the host: which physical page holds which tokens
// of which request.  No device memory is touched here; the tensors that the
// page ids index are owned by the engine.
//
// Model (after the reference's pool, src/engine/kvcache/pool.rs:128-321):
//  * a page holds `page_size` token slots; flat slot = page * page_size + offset;
//  * page 0 of every group is a sink that is never handed out (padding rows of
//    a replayed graph write to it and read it); usable ids are 1..N;
//  * free pages form a LIFO stack: a fresh pool of 10 hands out 10, 9, 8, ...
//    (pool.rs:271-288), so reuse is deterministic.
// Beyond the reference: layers with different needs form GROUPS with pages of
// their own.  A group either keeps all keys of a request or only a window of
// the last `window` positions; pages that the window has passed are given back
// while the request still runs.  A request may hold a PROMISE of pages
// (reserved at admission, taken later): a page that is promised to one request
// is never handed to another, so a running request cannot run out of pages.
// Fixed-size state slots (one per live request, slot 0 is the sink for padding
// rows) are handed out and taken back together with the pages.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200 {

struct GroupSpec {
  int page_size = 16;
  int num_pages = 0;   // usable pages, ids 1..num_pages
  int window = 0;      // 0: all keys are kept; W > 0: only keys j with p - W < j <= p are read
};

enum class Acquire : int { Ready = 0, DeferredMemory = 1, Impossible = 2, DeferredSlots = 3 };

class PagePool {
 public:
  explicit PagePool(int num_pages);
  int alloc();                 // -1 when empty
  bool release(int page);      // false: not held (freeing twice or a foreign id is refused)
  int free_count() const { return static_cast<int>(free_.size()); }
  int num_pages() const { return num_pages_; }
  bool is_held(int page) const { return page >= 1 && page <= num_pages_ && held_[page]; }
  const std::vector<int>& free_list() const { return free_; }

 private:
  int num_pages_;
  std::vector<int> free_;
  std::vector<uint8_t> held_;
};

struct GroupPages {
  std::vector<int> table;   // logical page -> physical id; 0 where nothing is held
  int first_live = 0;       // logical pages below this one were given back
  int held = 0;             // pages held now
  int promised = 0;         // pages that may still be taken without asking
  int promise_cap = 0;      // held + promised never needs to exceed this (0: no promise was made)
};

struct RequestCache {
  int64_t id = 0;
  int length = 0;           // tokens whose keys and values are in the cache
  int state_slot = 0;
  std::vector<GroupPages> groups;
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, int num_state_slots);

  int num_groups() const { return static_cast<int>(specs_.size()); }
  const GroupSpec& group(int g) const { return specs_.at(g); }
  int free_pages(int g) const { return pools_.at(g).free_count(); }
  int unpromised_pages(int g) const { return pools_.at(g).free_count() - promised_total_.at(g); }
  int free_state_slots() const { return static_cast<int>(free_slots_.size()); }
  int live_requests() const { return static_cast<int>(requests_.size()); }
  bool has(int64_t id) const { return requests_.count(id) != 0; }

  // Pages that a request of `capacity_tokens` needs in group g when no step
  // brings it more than `max_step_tokens` tokens.
  int pages_needed(int g, int capacity_tokens, int max_step_tokens) const;

  // Admission with a promise for the request's whole life (reference:
  // src/scheduler/prefill.rs:191-195, src/engine/kvcache/naive.rs:18-41).
  Acquire acquire(int64_t id, int capacity_tokens, int max_step_tokens);
  // Admission without a promise: pages are taken as the request grows.
  Acquire open(int64_t id);

  // Make pages cover positions [0, new_length) (windowed groups: from the
  // first live page).  False, and nothing changed, if a group cannot give them.
  bool grow(int64_t id, int new_length);
  // The same for several requests at once: either all of them get their pages or nothing changes.  Returns -1, or
  // the index of the first request for which the free pages do not reach (those before it would fit).
  int grow_all(const std::vector<int64_t>& ids, const std::vector<int>& new_lengths);
  // The request now holds `new_length` tokens; windowed groups give back the
  // pages that no later query can read.
  void advance(int64_t id, int new_length);
  // Give back everything.  Returns false for an unknown id (a second release is a no-op).
  bool release(int64_t id);

  int length(int64_t id) const { return requests_.at(id).length; }
  int state_slot(int64_t id) const { return requests_.at(id).state_slot; }
  const std::vector<int>& block_table(int64_t id, int g) const { return requests_.at(id).groups.at(g).table; }
  int first_live_page(int64_t id, int g) const { return requests_.at(id).groups.at(g).first_live; }
  int pages_held(int64_t id, int g) const { return requests_.at(id).groups.at(g).held; }
  // Flat slot of `position`; -1 if the page is not held.
  int slot_of(int64_t id, int g, int position) const;

  // Empty if every page is either free once or held once by one request, the
  // sink is nowhere, and the counters agree; else what is wrong.
  std::string check() const;

 private:
  Acquire admit(int64_t id, const std::vector<int>& promise);
  std::vector<GroupSpec> specs_;
  std::vector<PagePool> pools_;
  std::vector<int> promised_total_;
  std::vector<int> free_slots_;
  int num_state_slots_;
  std::unordered_map<int64_t, RequestCache> requests_;
};

}  // namespace b200
