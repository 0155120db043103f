// Host-side LPT (longest-processing-time-first) minibatch packer.
//
// Behavioural counterpart of the reference's numba-compiled packer
// (batch_packer.py:12-187): sequences are sorted longest first; each minibatch takes the
// largest prefix of the remaining sequences that an LPT schedule over `num_ranks` bins can
// place without any bin exceeding `max_tokens`; the prefix size is found by binary search
// over a feasibility check that uses a binary min-heap of per-rank loads.
//
// Differences by design (not by accident):
//  * the sort is a stable descending sort (ties keep ascending original index), so the result
//    is a pure function of the input on every platform;
//  * one call computes the assignment of EVERY rank, so a loader that needs all ranks (tests,
//    the single-process simulator) pays for one schedule instead of `num_ranks` schedules.
//
// C ABI, no Python headers: loaded with ctypes.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

namespace {

struct Heap {
  // 1-indexed binary min-heap over per-rank loads; id[] tracks which rank sits in each slot.
  std::vector<int64_t> load;
  std::vector<int64_t> id;
  int64_t n;
  explicit Heap(int64_t ranks) : load(ranks + 1, 0), id(ranks + 1, 0), n(ranks) {}
  void reset() {
    std::fill(load.begin(), load.end(), 0);
    for (int64_t i = 0; i <= n; ++i) id[i] = i - 1;
  }
  inline void sift_root() {
    int64_t u = 1;
    while ((u << 1) <= n) {
      int64_t v = u << 1;
      int64_t r = v | 1;
      if (r <= n && load[r] < load[v]) v = r;
      if (load[u] <= load[v]) break;
      std::swap(load[u], load[v]);
      std::swap(id[u], id[v]);
      u = v;
    }
  }
};

// True when LPT places lens[0..count) (already sorted descending) without overflow.
bool lpt_fits(Heap& h, const int64_t* lens, int64_t count, int64_t max_tokens) {
  h.reset();
  for (int64_t i = 0; i < count; ++i) {
    h.load[1] += lens[i];
    if (h.load[1] > max_tokens) return false;
    h.sift_root();
  }
  return true;
}

}  // namespace

extern "C" {

// Packs `n` sequence lengths for all ranks.
//   out_rank[i]      : rank that owns sequence i
//   out_minibatch[i] : minibatch index of sequence i
// Returns the number of minibatches (0 for an empty batch, -1 on bad arguments).
// A rank that owns no sequence of some minibatch gets a padding entry in the Python wrapper.
int64_t mtb200_lpt_pack(const int64_t* lengths, int64_t n, int64_t max_tokens, int64_t num_ranks,
                        int64_t* out_rank, int64_t* out_minibatch) {
  if (n < 0 || num_ranks <= 0) return -1;
  if (n == 0) return 0;
  std::vector<int64_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(),
                   [&](int64_t a, int64_t b) { return lengths[a] > lengths[b]; });
  std::vector<int64_t> sorted(n), csum(n);
  int64_t acc = 0;
  for (int64_t i = 0; i < n; ++i) {
    sorted[i] = lengths[order[i]];
    acc += sorted[i];
    csum[i] = acc;
  }
  Heap heap(num_ranks);
  int64_t start = 0, n_mb = 0;
  while (start < n) {
    const int64_t remaining = n - start;
    const int64_t base = start > 0 ? csum[start - 1] : 0;
    // Upper bound on the prefix: total tokens cannot exceed the capacity of all ranks.
    const int64_t cap = base + max_tokens * num_ranks;
    const int64_t ub = std::upper_bound(csum.begin() + start, csum.end(), cap) - (csum.begin() + start);
    int64_t left = 1;
    int64_t right = std::min(remaining + 1, ub + 1);
    while (right - left > 1) {
      const int64_t mid = (left + right) / 2;
      if (lpt_fits(heap, sorted.data() + start, mid, max_tokens)) left = mid; else right = mid;
    }
    int64_t take = left;
    if (take < num_ranks && take < remaining) {
      // Prefer giving every rank one sequence when that still fits.
      const int64_t want = std::min(num_ranks, remaining);
      if (lpt_fits(heap, sorted.data() + start, want, max_tokens)) take = want;
    }
    heap.reset();
    for (int64_t i = 0; i < take; ++i) {
      heap.load[1] += sorted[start + i];
      out_rank[order[start + i]] = heap.id[1];
      out_minibatch[order[start + i]] = n_mb;
      heap.sift_root();
    }
    ++n_mb;
    start += take;
  }
  return n_mb;
}

// Cost-aware LPT. Same outer search as mtb200_lpt_pack (longest first, largest prefix that fits),
// but ranks are balanced on an estimated COMPUTE cost  len * (1 + len / cost_len)  instead of on
// tokens: the linear term stands for the GEMMs, the quadratic one for causal attention, and
// `cost_len` is the sequence length at which both cost the same. The token budget stays a hard
// per-rank limit. The global batch (hence the gradient) is unchanged; only which rank processes
// which sample differs, so the slowest rank of a step is less slow.
int64_t mtb200_lpt_pack_cost(const int64_t* lengths, int64_t n, int64_t max_tokens, int64_t num_ranks, double cost_len,
                             int64_t* out_rank, int64_t* out_minibatch) {
  if (n < 0 || num_ranks <= 0 || !(cost_len > 0)) return -1;
  if (n == 0) return 0;
  std::vector<int64_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return lengths[a] > lengths[b]; });
  std::vector<int64_t> sorted(n), csum(n);
  int64_t acc = 0;
  for (int64_t i = 0; i < n; ++i) { sorted[i] = lengths[order[i]]; acc += sorted[i]; csum[i] = acc; }
  auto cost = [&](int64_t len) { return static_cast<double>(len) * (1.0 + static_cast<double>(len) / cost_len); };
  // binary min-heap over (cost, rank) with the token load carried along
  std::vector<double> hc(num_ranks + 1);
  std::vector<int64_t> ht(num_ranks + 1), hid(num_ranks + 1);
  auto reset = [&]() { for (int64_t i = 0; i <= num_ranks; ++i) { hc[i] = 0.0; ht[i] = 0; hid[i] = i - 1; } };
  auto sift = [&]() {
    int64_t u = 1;
    while ((u << 1) <= num_ranks) {
      int64_t v = u << 1, r = v | 1;
      if (r <= num_ranks && hc[r] < hc[v]) v = r;
      if (hc[u] <= hc[v]) break;
      std::swap(hc[u], hc[v]); std::swap(ht[u], ht[v]); std::swap(hid[u], hid[v]);
      u = v;
    }
  };
  // places `count` sequences from `first`; returns false when the cheapest rank would overflow its
  // token budget (a sequence alone on an empty rank always passes, like the token packer)
  auto place = [&](int64_t first, int64_t count, bool record, int64_t mb) {
    reset();
    for (int64_t i = 0; i < count; ++i) {
      const int64_t len = sorted[first + i];
      if (ht[1] > 0 && ht[1] + len > max_tokens) return false;
      if (record) { out_rank[order[first + i]] = hid[1]; out_minibatch[order[first + i]] = mb; }
      ht[1] += len;
      hc[1] += cost(len);
      sift();
    }
    return true;
  };
  int64_t start = 0, n_mb = 0;
  while (start < n) {
    const int64_t remaining = n - start;
    const int64_t base = start > 0 ? csum[start - 1] : 0;
    const int64_t ub = std::upper_bound(csum.begin() + start, csum.end(), base + max_tokens * num_ranks) - (csum.begin() + start);
    int64_t left = 1, right = std::min(remaining + 1, ub + 1);
    while (right - left > 1) {
      const int64_t mid = (left + right) / 2;
      if (place(start, mid, false, 0)) left = mid; else right = mid;
    }
    int64_t take = left;
    if (take < num_ranks && take < remaining) {
      const int64_t want = std::min(num_ranks, remaining);
      if (place(start, want, false, 0)) take = want;
    }
    place(start, take, true, n_mb);
    ++n_mb;
    start += take;
  }
  return n_mb;
}

// Greedy first-come packer kept for comparison tests (reference sampler.py:41-95): walks the
// sequences in the given order, always adding to the least-loaded rank of the open minibatch
// and opening a new minibatch when even that rank would overflow.
int64_t mtb200_greedy_pack(const int64_t* lengths, int64_t n, int64_t max_tokens, int64_t num_ranks,
                           int64_t* out_rank, int64_t* out_minibatch) {
  if (n < 0 || num_ranks <= 0) return -1;
  std::vector<int64_t> loads(num_ranks, 0);
  int64_t mb = 0;
  bool any = false;
  for (int64_t i = 0; i < n; ++i) {
    int64_t best = std::min_element(loads.begin(), loads.end()) - loads.begin();
    if (loads[best] + lengths[i] > max_tokens) {
      // Close the open minibatch unless it is still empty (an over-length first sample).
      if (*std::max_element(loads.begin(), loads.end()) > 0) ++mb;
      std::fill(loads.begin(), loads.end(), 0);
      best = 0;
    }
    loads[best] += lengths[i];
    out_rank[i] = best;
    out_minibatch[i] = mb;
    any = true;
  }
  return any ? mb + 1 : 0;
}

}  // extern "C"
