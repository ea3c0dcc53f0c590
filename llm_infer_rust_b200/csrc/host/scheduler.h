// Request scheduler: admits requests, cuts prompts into portions under a token
// budget, decodes, finishes and frees.  It decides; the engine executes.
//
// Policy (after the reference's serial scheduler, src/scheduler/scheduler.rs:225-274,
// src/scheduler/prefill.rs:163-293, with one mixed batch instead of two forwards):
//  * every decoding request gets one token in every step;
//  * the token budget counts prompt tokens only; requests whose prompt is not
//    yet through go on first (continuation first), then waiting requests are
//    admitted in arrival order while rows and budget are left; a prompt longer
//    than what is left of the budget is cut there and goes on in the next step;
//  * at admission a request is promised the pages of its whole life,
//    capacity = min(prompt + max_tokens - 1, max_seq_len) tokens
//    (prefill.rs:191-195: the last sampled token never enters the cache);
//    WHEN PAGES RUN OUT the request at the head of the queue waits (and
//    everything behind it); nothing that runs is ever pre-empted or swapped;
//    a request that needs more pages than the pool has is aborted;
//  * finish: Stop on an end-of-sequence id (unless ignore_eos), Length when
//    max_tokens outputs exist or the sequence reaches max_seq_len
//    (scheduler.rs:570-578); the finishing token is emitted; pages and the
//    state slot are given back at once;
//  * a step that needs no decision can be planned before the step before it has reported its tokens
//    (successor(); after the reference's overlap of host and device work, scheduler.rs:935-1038): when
//    nothing waits, every running request sampled in the step and none of them can end by length, the
//    next step is one decoded token for each of them.  A request that ends on a stop id (or is aborted)
//    while its successor step already runs stays in that step as a dead row; commit_step drops its token.
#pragma once
#include <cstdint>
#include <deque>
#include <unordered_set>
#include <vector>

#include "page_cache.h"

namespace b200 {

struct SamplingParams {
  float temperature = 0.0f;   // <= 0: greedy
  int top_k = -1;             // <= 0: off
  float top_p = 1.0f;         // 0: greedy; outside [0, 1]: 1
  bool ignore_eos = false;
  int max_tokens = 1024;      // at least 1
  uint64_t seed = 0;
  SamplingParams normalized() const;
};

enum class Status : int { Waiting = 0, Prefilling = 1, Decoding = 2, Finished = 3 };
enum class FinishReason : int { None = 0, Stop = 1, Length = 2, Abort = 3, Error = 4 };

struct OutputToken {
  int64_t uid;
  int token;          // -1 for Abort / Error
  bool finished;
  FinishReason reason;
};

struct PlanEntry {
  int64_t uid;
  int start;          // position of the first token of this portion
  int count;
  bool sample;        // the last token of the portion yields the request's next token
  int output_index;   // index of that token among the request's outputs
};

struct StepPlan {
  std::vector<PlanEntry> entries;
  int prefill_tokens = 0;
  int decode_rows = 0;
};

struct SchedulerOptions {
  int max_running_req = 256;
  int max_seq_len = 8192;
  int max_batch_tokens = 8192;   // prompt tokens per step; <= 0: no limit and no cutting
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, SchedulerOptions options, std::vector<int> eos_ids);

  int64_t add_request(std::vector<int> prompt, SamplingParams params);
  bool abort_request(int64_t uid);
  bool is_idle() const { return pending_.empty() && running_.empty() && outbox_.empty(); }

  StepPlan plan_step();
  // The step after `plan`, if it can be known before `plan` is committed (see above); else no entries.  Its
  // entries stand in the order of `plan`'s, so the tokens sampled by `plan` are its inputs row by row.
  StepPlan successor(const StepPlan& plan) const;
  // Tokens of a planned portion, to hand to the engine.
  std::vector<int> tokens_of(const PlanEntry& e) const;
  SamplingParams params_of(int64_t uid) const;
  // `sampled` holds one token for each entry with sample == true, in order (also for entries whose request
  // is gone by now: those tokens are dropped).
  std::vector<OutputToken> commit_step(const StepPlan& plan, const std::vector<int>& sampled);
  // The step failed: every request in it finishes with Error and frees its pages.
  std::vector<OutputToken> fail_step(const StepPlan& plan);
  // The step could not even be built (nothing of it ran): requests that `plan` admitted give back what they were
  // promised and return to the head of the queue in their old order; the others stay as they were.  Returns how
  // many went back (reference: src/scheduler/prefill.rs:65-71, :119-129).
  int rollback_step(const StepPlan& plan);
  // Results that arose outside a step (aborts at submission or admission).
  std::vector<OutputToken> drain_outbox();

  int num_pending() const { return static_cast<int>(pending_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  Status status_of(int64_t uid) const;

 private:
  struct Request {
    int64_t uid;
    std::vector<int> tokens;   // prompt, then outputs
    int prompt_len;
    int cursor = 0;            // tokens already given to the engine
    int output_len = 0;
    Status status = Status::Waiting;
    SamplingParams params;
  };
  Request* find_running(int64_t uid);
  const Request* find_any(int64_t uid) const;
  void finish(int64_t uid);

  CacheManager* cache_;
  SchedulerOptions opt_;
  std::unordered_set<int> eos_;
  int64_t next_uid_ = 1;
  std::deque<Request> pending_;
  std::vector<Request> running_;
  std::vector<OutputToken> outbox_;
};

}  // namespace b200
