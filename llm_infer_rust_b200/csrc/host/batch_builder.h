// Flattens one step's rows into the integer arrays that the kernels read.
//
// A row is (request, its next `count` tokens); a row of one token is a decode
// row, a longer one a portion of a prompt; both kinds may stand side by side.
// Everything lands in ONE int32 buffer (pinned by the caller, copied to the
// device in one transfer); `BatchLayout` says where each array starts.
// The arrays follow the reference's batch tensors (src/engine/batch_context.rs:216-304:
// input ids, positions, write locations, cumulative query lengths, prefix
// lengths, block table, logits indices) with one set of write slots and one
// block table per cache group.
#pragma once
#include <cstdint>
#include <vector>

#include "page_cache.h"

namespace b200 {

struct BatchLayout {
  int num_tokens = 0;
  int num_rows = 0;        // rows in the arrays (real rows, then padding rows)
  int num_real_rows = 0;
  int num_decode = 0;      // rows of exactly one token
  int num_prefill = 0;     // rows of more than one token
  int num_logits = 0;
  int max_q_len = 0;
  int max_kv_len = 0;
  int off_tokens = 0, off_positions = 0, off_row_of_token = 0;
  int off_cu_q = 0, off_kv_len = 0, off_prefix_len = 0, off_state_slot = 0;
  int off_decode_rows = 0, off_prefill_rows = 0, off_logit_rows = 0;
  std::vector<int> off_slots;     // per group: write slot of every token
  std::vector<int> off_table;     // per group: block table [num_rows, table_width]
  std::vector<int> table_width;   // per group
  int total_ints = 0;
};

struct BatchRequest {
  std::vector<int64_t> ids;       // one per row
  std::vector<int> counts;        // tokens per row (>= 1)
  std::vector<int> tokens;        // all rows' tokens, concatenated
  std::vector<int> want_counts;   // per row: how many positions' logits are wanted
  std::vector<int> want_index;    // concatenated indices within the row's tokens
  int pad_rows_to = 0;            // > 0: add one-token padding rows (sink page, state slot 0) up to this many rows
  std::vector<int> fixed_table_width;   // per group; empty: as narrow as this batch allows
};

// Number of int32 the buffer must hold, without writing anything.
BatchLayout plan_batch(const CacheManager& cache, const BatchRequest& req);
// Fill `out` (capacity in int32).  Pages must already cover every row
// (CacheManager::grow); throws if a token has no page to be written to.
BatchLayout build_batch(const CacheManager& cache, const BatchRequest& req, int32_t* out,
                        int64_t capacity);

}  // namespace b200
