#include "scheduler.h"

#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace b200 {

SamplingParams SamplingParams::normalized() const {
  // src/engine/sampling.rs:31-41: max_tokens at least 1, an invalid top_p becomes 1.
  SamplingParams p = *this;
  p.max_tokens = std::max(p.max_tokens, 1);
  if (!(std::isfinite(p.top_p) && p.top_p >= 0.0f && p.top_p <= 1.0f)) p.top_p = 1.0f;
  return p;
}

Scheduler::Scheduler(CacheManager* cache, SchedulerOptions options, std::vector<int> eos_ids)
    : cache_(cache), opt_(options), eos_(eos_ids.begin(), eos_ids.end()) {
  if (cache == nullptr) throw std::invalid_argument("the scheduler needs a cache manager");
  if (opt_.max_running_req <= 0) throw std::invalid_argument("max_running_req must be positive");
  if (opt_.max_seq_len <= 0) throw std::invalid_argument("max_seq_len must be positive");
}

int64_t Scheduler::add_request(std::vector<int> prompt, SamplingParams params) {
  int64_t uid = next_uid_++;
  // An empty prompt (prefill.rs:180-184) or one beyond max_seq_len (scheduler.rs:168-170) is aborted.
  if (prompt.empty() || static_cast<int>(prompt.size()) > opt_.max_seq_len) {
    outbox_.push_back({uid, -1, true, FinishReason::Abort});
    return uid;
  }
  Request r;
  r.uid = uid;
  r.prompt_len = static_cast<int>(prompt.size());
  r.tokens = std::move(prompt);
  r.params = params.normalized();
  pending_.push_back(std::move(r));
  return uid;
}

Scheduler::Request* Scheduler::find_running(int64_t uid) {
  for (auto& r : running_) if (r.uid == uid) return &r;
  return nullptr;
}

const Scheduler::Request* Scheduler::find_any(int64_t uid) const {
  for (const auto& r : running_) if (r.uid == uid) return &r;
  for (const auto& r : pending_) if (r.uid == uid) return &r;
  return nullptr;
}

Status Scheduler::status_of(int64_t uid) const {
  const Request* r = find_any(uid);
  return r ? r->status : Status::Finished;
}

SamplingParams Scheduler::params_of(int64_t uid) const {
  const Request* r = find_any(uid);
  if (!r) throw std::invalid_argument("unknown request");
  return r->params;
}

void Scheduler::finish(int64_t uid) {
  cache_->release(uid);
  running_.erase(std::remove_if(running_.begin(), running_.end(),
                                [uid](const Request& r) { return r.uid == uid; }),
                 running_.end());
}

bool Scheduler::abort_request(int64_t uid) {
  for (auto it = pending_.begin(); it != pending_.end(); ++it) {
    if (it->uid == uid) {
      pending_.erase(it);
      outbox_.push_back({uid, -1, true, FinishReason::Abort});
      return true;
    }
  }
  if (find_running(uid)) {
    finish(uid);
    outbox_.push_back({uid, -1, true, FinishReason::Abort});
    return true;
  }
  return false;
}

std::vector<OutputToken> Scheduler::drain_outbox() {
  std::vector<OutputToken> out;
  out.swap(outbox_);
  return out;
}

StepPlan Scheduler::plan_step() {
  StepPlan plan;
  const bool limited = opt_.max_batch_tokens > 0;
  int budget = limited ? opt_.max_batch_tokens : 0;
  const int step_bound = limited ? opt_.max_batch_tokens : opt_.max_seq_len;

  for (auto& r : running_) {
    if (r.status != Status::Decoding) continue;
    plan.entries.push_back({r.uid, r.cursor, 1, true, r.output_len});
    plan.decode_rows += 1;
  }
  for (auto& r : running_) {
    if (r.status != Status::Prefilling) continue;
    int remaining = r.prompt_len - r.cursor;
    int n = limited ? std::min(remaining, budget) : remaining;
    if (n <= 0) break;
    plan.entries.push_back({r.uid, r.cursor, n, r.cursor + n == r.prompt_len, r.output_len});
    plan.prefill_tokens += n;
    if (limited) budget -= n;
  }
  while (!pending_.empty() && static_cast<int>(running_.size()) < opt_.max_running_req &&
         (!limited || budget > 0)) {
    Request& head = pending_.front();
    int capacity = std::min(head.prompt_len + head.params.max_tokens - 1, opt_.max_seq_len);
    Acquire got = cache_->acquire(head.uid, capacity, step_bound);
    if (got == Acquire::Impossible) {
      outbox_.push_back({head.uid, -1, true, FinishReason::Abort});
      pending_.pop_front();
      continue;
    }
    if (got != Acquire::Ready) break;   // the head of the queue waits, and all behind it
    Request r = std::move(head);
    pending_.pop_front();
    r.status = Status::Prefilling;
    int n = limited ? std::min(r.prompt_len, budget) : r.prompt_len;
    plan.entries.push_back({r.uid, 0, n, n == r.prompt_len, 0});
    plan.prefill_tokens += n;
    if (limited) budget -= n;
    running_.push_back(std::move(r));
  }
  return plan;
}

StepPlan Scheduler::successor(const StepPlan& plan) const {
  StepPlan next;
  if (!pending_.empty() || plan.entries.size() != running_.size()) return next;
  for (const PlanEntry& e : plan.entries) {
    const Request* r = nullptr;
    for (const Request& q : running_)
      if (q.uid == e.uid) { r = &q; break; }
    // after `plan`: one more output, one more token in the sequence
    if (!r || !e.sample || e.output_index + 1 >= r->params.max_tokens || e.start + e.count + 1 >= opt_.max_seq_len)
      return StepPlan();
    next.entries.push_back({e.uid, e.start + e.count, 1, true, e.output_index + 1});
  }
  next.decode_rows = static_cast<int>(next.entries.size());
  return next;
}

std::vector<int> Scheduler::tokens_of(const PlanEntry& e) const {
  const Request* r = find_any(e.uid);
  if (!r) throw std::invalid_argument("plan entry of an unknown request");
  if (e.start < 0 || e.start + e.count > static_cast<int>(r->tokens.size()))
    throw std::out_of_range("plan entry outside the request's tokens");
  return std::vector<int>(r->tokens.begin() + e.start, r->tokens.begin() + e.start + e.count);
}

std::vector<OutputToken> Scheduler::commit_step(const StepPlan& plan, const std::vector<int>& sampled) {
  std::vector<OutputToken> out;
  size_t next = 0;
  for (const PlanEntry& e : plan.entries) {
    Request* r = find_running(e.uid);
    if (!r) {           // finished or aborted while the step ran: its token is dropped
      if (e.sample) {
        if (next >= sampled.size()) throw std::invalid_argument("fewer sampled tokens than sampling rows");
        ++next;
      }
      continue;
    }
    r->cursor = e.start + e.count;
    if (!e.sample) continue;
    if (next >= sampled.size()) throw std::invalid_argument("fewer sampled tokens than sampling rows");
    int token = sampled[next++];
    r->tokens.push_back(token);
    r->output_len += 1;
    r->status = Status::Decoding;
    FinishReason reason = FinishReason::None;
    if (!r->params.ignore_eos && eos_.count(token)) reason = FinishReason::Stop;
    else if (r->output_len >= r->params.max_tokens ||
             static_cast<int>(r->tokens.size()) >= opt_.max_seq_len) reason = FinishReason::Length;
    bool finished = reason != FinishReason::None;
    out.push_back({e.uid, token, finished, reason});
    if (finished) finish(e.uid);
  }
  if (next != sampled.size()) throw std::invalid_argument("more sampled tokens than sampling rows");
  return out;
}

int Scheduler::rollback_step(const StepPlan& plan) {
  int moved = 0;
  // last admitted first, each to the front: the queue ends up in arrival order again
  for (auto e = plan.entries.rbegin(); e != plan.entries.rend(); ++e) {
    if (e->start != 0) continue;
    auto it = std::find_if(running_.begin(), running_.end(), [&](const Request& r) { return r.uid == e->uid; });
    if (it == running_.end() || it->status != Status::Prefilling || it->cursor != 0) continue;
    Request r = std::move(*it);
    running_.erase(it);
    cache_->release(r.uid);
    r.status = Status::Waiting;
    pending_.push_front(std::move(r));
    ++moved;
  }
  return moved;
}

std::vector<OutputToken> Scheduler::fail_step(const StepPlan& plan) {
  std::vector<OutputToken> out;
  for (const PlanEntry& e : plan.entries) {
    if (!find_running(e.uid)) continue;
    finish(e.uid);
    out.push_back({e.uid, -1, true, FinishReason::Error});
  }
  return out;
}

}  // namespace b200
