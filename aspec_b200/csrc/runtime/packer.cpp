// Work-aware packing of whole documents into one row per data-parallel rank, plus the run-length
// loss-mask helpers the scheduler needs.
//
// Rule (same behaviour as aspec/controller/packing.py:87-167 in the reference): each of the dp rows is
// seeded with one of the dp oldest samples; the remaining samples are visited by useful-anchor
// density (ties: more work, longer, older) and each goes to the row it fills tightest; rows are then
// ordered longest first.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

extern "C" {

// row_of[i] = rank row (after longest-first ordering) of sample i, or -1 when not selected.
// order_in_row[i] = position of sample i inside its row.  Returns 0 ok, 1 not enough samples,
// -1 bad arguments, -2 a sample can never fit.
int ab_pack_rows(int n, const int* lengths, const long long* useful, int dp, int max_seq, int max_selected,
                 int* row_of, int* order_in_row, long long* packed_tokens, long long* useful_total) {
  if (dp <= 0 || max_seq <= 0 || n < 0) return -1;
  if (max_selected >= 0 && max_selected < dp) return -1;
  for (int i = 0; i < n; ++i)
    if (lengths[i] <= 0 || lengths[i] > max_seq) return -2;
  if (n < dp) return 1;
  std::vector<std::vector<int>> rows(dp);
  std::vector<long long> used(dp);
  int selected = dp;
  for (int r = 0; r < dp; ++r) { rows[r].push_back(r); used[r] = lengths[r]; }
  std::vector<int> cand(n - dp);
  std::iota(cand.begin(), cand.end(), dp);
  std::sort(cand.begin(), cand.end(), [&](int a, int b) {
    // density compared exactly as cross products: useful[a]/len[a] > useful[b]/len[b]
    const __int128 da = (__int128)useful[a] * lengths[b], db = (__int128)useful[b] * lengths[a];
    if (da != db) return da > db;
    if (useful[a] != useful[b]) return useful[a] > useful[b];
    if (lengths[a] != lengths[b]) return lengths[a] > lengths[b];
    return a < b;
  });
  for (int idx : cand) {
    if (max_selected >= 0 && selected >= max_selected) break;
    int best = -1;
    for (int r = 0; r < dp; ++r) {
      if (used[r] + lengths[idx] > max_seq) continue;
      if (best < 0) { best = r; continue; }
      const long long slack_r = max_seq - used[r] - lengths[idx], slack_b = max_seq - used[best] - lengths[idx];
      if (slack_r < slack_b || (slack_r == slack_b && used[r] < used[best])) best = r;
    }
    if (best < 0) continue;
    rows[best].push_back(idx);
    used[best] += lengths[idx];
    ++selected;
  }
  std::vector<int> order(dp);
  std::iota(order.begin(), order.end(), 0);
  std::sort(order.begin(), order.end(), [&](int a, int b) { return used[a] != used[b] ? used[a] > used[b] : a < b; });
  for (int i = 0; i < n; ++i) { row_of[i] = -1; order_in_row[i] = -1; }
  long long tokens = 0, work = 0;
  for (int rank = 0; rank < dp; ++rank) {
    const auto& row = rows[order[rank]];
    for (size_t j = 0; j < row.size(); ++j) {
      row_of[row[j]] = rank;
      order_in_row[row[j]] = (int)j;
      tokens += lengths[row[j]];
      work += useful[row[j]];
    }
  }
  *packed_tokens = tokens;
  *useful_total = work;
  return 0;
}

// Run-length loss mask: alternating run lengths that start with an unsupervised run.
// Supervised anchor starts whose whole block stays inside the sample.
long long ab_count_anchor_starts(const long long* runs, int n_runs, long long sample_length, int block_size) {
  if (sample_length <= 0 || block_size <= 0) return 0;
  const long long prefix = std::max<long long>(sample_length - block_size + 1, 0);
  long long cursor = 0, count = 0;
  for (int i = 0; i < n_runs; ++i) {
    if (runs[i] < 0) return -1;
    const long long end = cursor + runs[i];
    if (i & 1) count += std::max<long long>(0, std::min(end, prefix) - std::min(cursor, prefix));
    cursor = end;
  }
  return count;
}

// Next-token supervision summed over the recurrent depths of an EAGLE draft.
long long ab_count_eagle_positions(const long long* runs, int n_runs, long long sample_length, int ttt_length) {
  long long cursor = 0, total = 0;
  for (int i = 0; i < n_runs; ++i) {
    if (runs[i] < 0) return -1;
    const long long end = cursor + runs[i];
    if (i & 1)
      for (int depth = 0; depth < ttt_length; ++depth)
        total += std::max<long long>(0, std::min(end, sample_length - 1) - std::max<long long>(cursor, depth));
    cursor = end;
  }
  return total;
}

// Expand runs into a 0/1 byte mask of `length` entries; returns the number written.
long long ab_expand_loss_mask(const long long* runs, int n_runs, unsigned char* mask, long long length) {
  long long cursor = 0;
  for (int i = 0; i < n_runs && cursor < length; ++i) {
    const long long end = std::min(length, cursor + runs[i]);
    for (long long j = cursor; j < end; ++j) mask[j] = (unsigned char)(i & 1);
    cursor = end;
  }
  for (long long j = cursor; j < length; ++j) mask[j] = 0;
  return cursor;
}

// Assistant-span loss mask on token ids: after every occurrence of `header` (plus `skip_after` tokens) mark
// tokens as supervised until `end` begins (or to the end of the sequence when no terminator follows).
// Returns the start of the last assistant span (0 when none).
long long ab_assistant_loss_mask(const long long* ids, long long n, const long long* header, int header_len,
                                 const long long* end, int end_len, int skip_after, unsigned char* out) {
  for (long long k = 0; k < n; ++k) out[k] = 0;
  if (header_len <= 0) return 0;
  long long i = 0, last_start = 0;
  while (i <= n - header_len) {
    bool match = true;
    for (int k = 0; k < header_len; ++k)
      if (ids[i + k] != header[k]) { match = false; break; }
    if (!match) { ++i; continue; }
    long long j = i + header_len + skip_after;
    last_start = j;
    bool found = false;
    while (end_len > 0 && j <= n - end_len) {
      bool e = true;
      for (int k = 0; k < end_len; ++k)
        if (ids[j + k] != end[k]) { e = false; break; }
      if (e) { found = true; break; }
      out[j] = 1;
      ++j;
    }
    if (!found) for (long long k = std::max<long long>(j, 0); k < n; ++k) out[k] = 1;
    i = j + std::max(end_len, 1);
  }
  return last_start;
}

}  // extern "C"
