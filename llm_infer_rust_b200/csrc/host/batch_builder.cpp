#include "batch_builder.h"

#include <algorithm>
#include <stdexcept>
#include <string>

namespace b200 {

static int align4(int n) { return (n + 3) & ~3; }

BatchLayout plan_batch(const CacheManager& cache, const BatchRequest& req) {
  const int real = static_cast<int>(req.ids.size());
  if (static_cast<int>(req.counts.size()) != real || static_cast<int>(req.want_counts.size()) != real)
    throw std::invalid_argument("ids, counts and want_counts must have one entry per row");
  BatchLayout L;
  L.num_real_rows = real;
  L.num_rows = std::max(real, req.pad_rows_to);
  const int pad = L.num_rows - real;
  int tokens = 0, wants = 0;
  for (int r = 0; r < real; ++r) {
    if (req.counts[r] <= 0) throw std::invalid_argument("a row must bring at least one token");
    if (!cache.has(req.ids[r])) throw std::invalid_argument("a row names a request that holds no cache");
    for (int q = 0; q < r; ++q)
      if (req.ids[q] == req.ids[r]) throw std::invalid_argument("a request may appear once in a step");
    int prefix = cache.length(req.ids[r]);
    tokens += req.counts[r];
    wants += req.want_counts[r];
    (req.counts[r] == 1 ? L.num_decode : L.num_prefill) += 1;
    L.max_q_len = std::max(L.max_q_len, req.counts[r]);
    L.max_kv_len = std::max(L.max_kv_len, prefix + req.counts[r]);
  }
  if (static_cast<int>(req.tokens.size()) != tokens) throw std::invalid_argument("tokens do not add up to the rows' counts");
  if (static_cast<int>(req.want_index.size()) != wants) throw std::invalid_argument("want_index does not add up to want_counts");
  if (pad > 0) { L.max_q_len = std::max(L.max_q_len, 1); L.max_kv_len = std::max(L.max_kv_len, 1); }
  L.num_decode += pad;
  L.num_tokens = tokens + pad;
  L.num_logits = wants + pad;

  const int G = cache.num_groups();
  if (!req.fixed_table_width.empty() && static_cast<int>(req.fixed_table_width.size()) != G)
    throw std::invalid_argument("fixed_table_width needs one entry per cache group");
  int off = 0;
  auto take = [&off](int n) { int at = off; off += align4(std::max(n, 1)); return at; };
  L.off_tokens = take(L.num_tokens);
  L.off_positions = take(L.num_tokens);
  L.off_row_of_token = take(L.num_tokens);
  L.off_cu_q = take(L.num_rows + 1);
  L.off_kv_len = take(L.num_rows);
  L.off_prefix_len = take(L.num_rows);
  L.off_state_slot = take(L.num_rows);
  L.off_decode_rows = take(L.num_decode);
  L.off_prefill_rows = take(L.num_prefill);
  L.off_logit_rows = take(L.num_logits);
  for (int g = 0; g < G; ++g) {
    int width = 1;
    if (!req.fixed_table_width.empty()) {
      width = req.fixed_table_width[g];
    } else {
      int P = cache.group(g).page_size;
      width = std::max(1, (L.max_kv_len + P - 1) / P);
    }
    L.table_width.push_back(width);
    L.off_slots.push_back(take(L.num_tokens));
    L.off_table.push_back(take(L.num_rows * width));
  }
  L.total_ints = off;
  return L;
}

BatchLayout build_batch(const CacheManager& cache, const BatchRequest& req, int32_t* out, int64_t capacity) {
  BatchLayout L = plan_batch(cache, req);
  if (L.total_ints > capacity) throw std::length_error("the batch buffer is too small for this step");
  std::fill(out, out + L.total_ints, 0);
  const int G = cache.num_groups();
  int t = 0, w = 0, n_dec = 0, n_pf = 0, n_logit = 0;
  out[L.off_cu_q] = 0;
  for (int r = 0; r < L.num_rows; ++r) {
    const bool real = r < L.num_real_rows;
    const int count = real ? req.counts[r] : 1;
    const int prefix = real ? cache.length(req.ids[r]) : 0;
    out[L.off_kv_len + r] = prefix + count;
    out[L.off_prefix_len + r] = prefix;
    out[L.off_state_slot + r] = real ? cache.state_slot(req.ids[r]) : 0;
    out[L.off_cu_q + r + 1] = t + count;
    if (count == 1) out[L.off_decode_rows + n_dec++] = r; else out[L.off_prefill_rows + n_pf++] = r;
    if (real) {
      for (int i = 0; i < req.want_counts[r]; ++i) {
        int idx = req.want_index[w++];
        if (idx < 0 || idx >= count) throw std::out_of_range("a wanted position lies outside its row");
        out[L.off_logit_rows + n_logit++] = t + idx;
      }
    } else {
      out[L.off_logit_rows + n_logit++] = t;
    }
    for (int g = 0; g < G; ++g) {
      const int width = L.table_width[g];
      int32_t* row = out + L.off_table[g] + static_cast<int64_t>(r) * width;
      if (real) {
        const std::vector<int>& table = cache.block_table(req.ids[r], g);
        const int P = cache.group(g).page_size;
        const int used = (prefix + count + P - 1) / P;
        if (used > width) throw std::length_error("a block table is wider than the batch allows");
        for (int lp = 0; lp < used && lp < static_cast<int>(table.size()); ++lp) row[lp] = table[lp];
      }
    }
    for (int i = 0; i < count; ++i, ++t) {
      out[L.off_tokens + t] = real ? req.tokens[t] : 0;
      out[L.off_positions + t] = prefix + i;
      out[L.off_row_of_token + t] = r;
      for (int g = 0; g < G; ++g) {
        int slot = 0;
        if (real) {
          slot = cache.slot_of(req.ids[r], g, prefix + i);
          if (slot < 0)
            throw std::runtime_error("token at position " + std::to_string(prefix + i) +
                                     " has no page to be written to in cache group " + std::to_string(g));
        }
        out[L.off_slots[g] + t] = slot;
      }
    }
  }
  return L;
}

}  // namespace b200
