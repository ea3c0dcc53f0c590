#include "page_cache.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace b200 {

static int ceil_div(int a, int b) { return (a + b - 1) / b; }

PagePool::PagePool(int num_pages) : num_pages_(num_pages), held_(num_pages + 1, 0) {
  if (num_pages < 0) throw std::invalid_argument("a pool cannot have a negative number of pages");
  free_.reserve(num_pages);
  for (int p = 1; p <= num_pages; ++p) free_.push_back(p);   // popped from the back: N, N-1, ...
}

int PagePool::alloc() {
  if (free_.empty()) return -1;
  int page = free_.back();
  free_.pop_back();
  held_[page] = 1;
  return page;
}

bool PagePool::release(int page) {
  if (page < 1 || page > num_pages_ || !held_[page]) return false;
  held_[page] = 0;
  free_.push_back(page);
  return true;
}

CacheManager::CacheManager(std::vector<GroupSpec> groups, int num_state_slots)
    : specs_(std::move(groups)), num_state_slots_(num_state_slots) {
  if (num_state_slots < 0) throw std::invalid_argument("negative number of state slots");
  for (const auto& s : specs_) {
    if (s.page_size <= 0) throw std::invalid_argument("page_size must be positive");
    if (s.window < 0) throw std::invalid_argument("window must not be negative");
    pools_.emplace_back(s.num_pages);
    promised_total_.push_back(0);
  }
  for (int s = num_state_slots; s >= 1; --s) free_slots_.push_back(s);   // handed out 1, 2, ...
}

int CacheManager::pages_needed(int g, int capacity_tokens, int max_step_tokens) const {
  const GroupSpec& s = specs_.at(g);
  int all = ceil_div(std::max(capacity_tokens, 0), s.page_size);
  if (s.window == 0) return all;
  // Live positions span at most [L - W + 1, L + step): W + step - 1 positions,
  // which touch at most ceil(that / P) + 1 pages.
  int span = s.window + std::max(max_step_tokens, 1) - 1;
  return std::min(all, ceil_div(span, s.page_size) + 1);
}

Acquire CacheManager::admit(int64_t id, const std::vector<int>& promise) {
  if (requests_.count(id)) throw std::invalid_argument("request id is already live");
  for (size_t g = 0; g < specs_.size(); ++g)
    if (promise[g] > specs_[g].num_pages) return Acquire::Impossible;
  if (num_state_slots_ == 0 || free_slots_.empty()) return Acquire::DeferredSlots;
  for (size_t g = 0; g < specs_.size(); ++g)
    if (promise[g] > unpromised_pages(static_cast<int>(g))) return Acquire::DeferredMemory;
  RequestCache rc;
  rc.id = id;
  rc.state_slot = free_slots_.back();
  free_slots_.pop_back();
  rc.groups.resize(specs_.size());
  for (size_t g = 0; g < specs_.size(); ++g) {
    rc.groups[g].promised = promise[g];
    rc.groups[g].promise_cap = promise[g];
    promised_total_[g] += promise[g];
  }
  requests_.emplace(id, std::move(rc));
  return Acquire::Ready;
}

Acquire CacheManager::acquire(int64_t id, int capacity_tokens, int max_step_tokens) {
  std::vector<int> promise(specs_.size());
  for (size_t g = 0; g < specs_.size(); ++g)
    promise[g] = pages_needed(static_cast<int>(g), capacity_tokens, max_step_tokens);
  return admit(id, promise);
}

Acquire CacheManager::open(int64_t id) { return admit(id, std::vector<int>(specs_.size(), 0)); }

bool CacheManager::grow(int64_t id, int new_length) {
  RequestCache& rc = requests_.at(id);
  // First see that every group can give what is asked, then take.
  std::vector<int> need(specs_.size(), 0);
  for (size_t g = 0; g < specs_.size(); ++g) {
    const GroupPages& gp = rc.groups[g];
    int want = ceil_div(new_length, specs_[g].page_size);
    int have = static_cast<int>(gp.table.size());
    need[g] = std::max(0, want - std::max(have, gp.first_live));
    int beyond_promise = std::max(0, need[g] - gp.promised);
    if (beyond_promise > unpromised_pages(static_cast<int>(g))) return false;
  }
  for (size_t g = 0; g < specs_.size(); ++g) {
    GroupPages& gp = rc.groups[g];
    int want = ceil_div(new_length, specs_[g].page_size);
    if (static_cast<int>(gp.table.size()) < want) gp.table.resize(want, 0);
    for (int lp = std::max(want - need[g], gp.first_live); lp < want; ++lp) {
      if (gp.table[lp] != 0) continue;
      int page = pools_[g].alloc();
      if (page < 0) throw std::logic_error("page accounting is broken: pool empty after the check");
      gp.table[lp] = page;
      gp.held += 1;
      if (gp.promised > 0) { gp.promised -= 1; promised_total_[g] -= 1; }
    }
  }
  return true;
}

int CacheManager::grow_all(const std::vector<int64_t>& ids, const std::vector<int>& new_lengths) {
  if (ids.size() != new_lengths.size()) throw std::invalid_argument("one length for every request");
  for (size_t i = 0; i < ids.size(); ++i)
    for (size_t j = 0; j < i; ++j)
      if (ids[j] == ids[i]) throw std::invalid_argument("a request appears twice in one step");
  std::vector<int> beyond(specs_.size(), 0);      // pages beyond the requests' own promises, taken so far
  for (size_t i = 0; i < ids.size(); ++i) {
    const RequestCache& rc = requests_.at(ids[i]);
    for (size_t g = 0; g < specs_.size(); ++g) {
      const GroupPages& gp = rc.groups[g];
      int want = ceil_div(new_lengths[i], specs_[g].page_size);
      int have = static_cast<int>(gp.table.size());
      int need = std::max(0, want - std::max(have, gp.first_live));
      beyond[g] += std::max(0, need - gp.promised);
      if (beyond[g] > unpromised_pages(static_cast<int>(g))) return static_cast<int>(i);
    }
  }
  for (size_t i = 0; i < ids.size(); ++i)
    if (!grow(ids[i], new_lengths[i])) throw std::logic_error("page accounting is broken: a checked growth failed");
  return -1;
}

void CacheManager::advance(int64_t id, int new_length) {
  RequestCache& rc = requests_.at(id);
  if (new_length < rc.length) throw std::invalid_argument("a request cannot shrink");
  rc.length = new_length;
  for (size_t g = 0; g < specs_.size(); ++g) {
    const GroupSpec& s = specs_[g];
    if (s.window == 0) continue;
    GroupPages& gp = rc.groups[g];
    // The next query sits at position >= new_length and reads keys j > new_length - W.
    int first_needed = new_length - s.window + 1;
    if (first_needed <= 0) continue;
    int keep_from = std::min(first_needed / s.page_size, static_cast<int>(gp.table.size()));
    for (int lp = gp.first_live; lp < keep_from; ++lp) {
      if (gp.table[lp] == 0) continue;
      pools_[g].release(gp.table[lp]);
      gp.table[lp] = 0;
      gp.held -= 1;
      // A request admitted with a promise needs a page again as it grows: the
      // promise goes back to it, so that nobody else is given this page's worth.
      if (gp.held + gp.promised < gp.promise_cap) {
        gp.promised += 1;
        promised_total_[g] += 1;
      }
    }
    gp.first_live = std::max(gp.first_live, keep_from);
  }
}

bool CacheManager::release(int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return false;
  RequestCache& rc = it->second;
  for (size_t g = 0; g < specs_.size(); ++g) {
    GroupPages& gp = rc.groups[g];
    for (int page : gp.table)
      if (page != 0) pools_[g].release(page);
    promised_total_[g] -= gp.promised;
  }
  free_slots_.push_back(rc.state_slot);
  requests_.erase(it);
  return true;
}

int CacheManager::slot_of(int64_t id, int g, int position) const {
  const GroupPages& gp = requests_.at(id).groups.at(g);
  int P = specs_[g].page_size;
  int lp = position / P;
  if (position < 0 || lp >= static_cast<int>(gp.table.size()) || gp.table[lp] == 0) return -1;
  return gp.table[lp] * P + position % P;
}

std::string CacheManager::check() const {
  std::ostringstream err;
  for (size_t g = 0; g < specs_.size(); ++g) {
    const PagePool& pool = pools_[g];
    std::vector<int> seen(pool.num_pages() + 1, 0);
    for (int page : pool.free_list()) {
      if (page < 1 || page > pool.num_pages()) { err << "group " << g << ": free list holds id " << page << "; "; continue; }
      if (pool.is_held(page)) err << "group " << g << ": page " << page << " is free and held; ";
      seen[page] += 1;
    }
    int promised = 0;
    for (const auto& kv : requests_) {
      const GroupPages& gp = kv.second.groups[g];
      int held = 0;
      for (size_t lp = 0; lp < gp.table.size(); ++lp) {
        int page = gp.table[lp];
        if (page == 0) continue;
        if (page < 1 || page > pool.num_pages()) { err << "group " << g << ": request " << kv.first << " holds id " << page << "; "; continue; }
        if (static_cast<int>(lp) < gp.first_live) err << "group " << g << ": request " << kv.first << " holds a page below its window; ";
        if (!pool.is_held(page)) err << "group " << g << ": page " << page << " of request " << kv.first << " is not marked held; ";
        seen[page] += 1;
        held += 1;
      }
      if (held != gp.held) err << "group " << g << ": request " << kv.first << " counts " << gp.held << " pages, holds " << held << "; ";
      if (gp.promised < 0) err << "group " << g << ": negative promise; ";
      promised += gp.promised;
    }
    for (int page = 1; page <= pool.num_pages(); ++page) {
      if (seen[page] == 0) err << "group " << g << ": page " << page << " is lost; ";
      if (seen[page] > 1) err << "group " << g << ": page " << page << " is held " << seen[page] << " times; ";
    }
    if (promised != promised_total_[g]) err << "group " << g << ": promises sum to " << promised << ", counter says " << promised_total_[g] << "; ";
    if (promised_total_[g] > pool.free_count()) err << "group " << g << ": more pages promised than free; ";
  }
  std::vector<int> slot_seen(num_state_slots_ + 1, 0);
  for (int s : free_slots_) if (s >= 1 && s <= num_state_slots_) slot_seen[s] += 1; else err << "bad free state slot " << s << "; ";
  for (const auto& kv : requests_) {
    int s = kv.second.state_slot;
    if (s >= 1 && s <= num_state_slots_) slot_seen[s] += 1; else err << "request " << kv.first << " holds state slot " << s << "; ";
  }
  for (int s = 1; s <= num_state_slots_; ++s)
    if (slot_seen[s] != 1) err << "state slot " << s << " is accounted " << slot_seen[s] << " times; ";
  return err.str();
}

}  // namespace b200
