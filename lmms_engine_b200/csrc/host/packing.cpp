// Host-side sequence packing and load-balancing cores (index based: callers keep the
// samples, this code only sees lengths and returns which sample goes into which pack).
//
//  * PackStream  - streaming packer with three policies:
//      0 next-fit   one open pack; flush it when the next sample does not fit (what the
//                   reference calls "first_fit": datasets/packing/online.py:8-40)
//      1 best-fit   K open packs, tightest fit wins, a pack is emitted once it is
//                   fill_threshold full, the fullest one is evicted under pressure
//                   (online.py:43-112)
//      2 balanced   K open packs, best-fit placement, move/swap local search across the
//                   open packs before the oldest is emitted (online.py:115-268)
//      3 first-fit  true first-fit over K open packs (extra strategy)
//  * offline_first_fit / offline_window - index groups for map-style datasets
//    (datasets/naive/multimodal_dataset.py:205-237)
//  * lpt_balance - longest-processing-time assignment of weighted items (video frames)
//    to ranks with a locality preference (parallel/vit_parallel/balance.py:22-195)
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <numeric>
#include <vector>

namespace {

struct Bucket {
  long total = 0;
  std::vector<long> ids;
  std::vector<long> lens;
};

struct PackStream {
  int policy;
  long capacity;
  int max_open;
  long fill_full;
  int max_swap_iters;
  long min_gain;
  std::vector<Bucket> open;
  // emitted packs wait here until the caller drains them
  std::vector<std::vector<long>> ready;

  void emit(size_t i) {
    ready.push_back(std::move(open[i].ids));
    open.erase(open.begin() + static_cast<long>(i));
  }

  int best_fit(long len) const {
    int best = -1;
    long best_rem = capacity + 1;
    for (size_t i = 0; i < open.size(); ++i) {
      long rem = capacity - open[i].total - len;
      if (rem >= 0 && rem < best_rem) {
        best_rem = rem;
        best = static_cast<int>(i);
      }
    }
    return best;
  }

  void balance() {
    const size_t n = open.size();
    if (n < 2) return;
    for (int iter = 0; iter < max_swap_iters; ++iter) {
      size_t hi = 0, lo = 0;
      for (size_t i = 1; i < n; ++i) {
        if (open[i].total > open[hi].total) hi = i;
        if (open[i].total < open[lo].total) lo = i;
      }
      const long gap = open[hi].total - open[lo].total;
      if (gap <= min_gain) break;
      // 1. single move hi -> lo
      int mv = -1;
      long best_gap = gap;
      for (size_t k = 0; k < open[hi].lens.size(); ++k) {
        const long l = open[hi].lens[k];
        if (open[lo].total + l > capacity) continue;
        const long g = std::labs((open[hi].total - l) - (open[lo].total + l));
        if (g < best_gap) { best_gap = g; mv = static_cast<int>(k); }
      }
      if (mv >= 0) {
        const long l = open[hi].lens[mv], id = open[hi].ids[mv];
        open[hi].lens.erase(open[hi].lens.begin() + mv);
        open[hi].ids.erase(open[hi].ids.begin() + mv);
        open[lo].lens.push_back(l);
        open[lo].ids.push_back(id);
        open[hi].total -= l;
        open[lo].total += l;
        continue;
      }
      // 2. pairwise swap
      int si = -1, sj = -1;
      best_gap = gap;
      for (size_t i = 0; i < open[hi].lens.size(); ++i) {
        for (size_t j = 0; j < open[lo].lens.size(); ++j) {
          const long a = open[hi].lens[i], b = open[lo].lens[j];
          if (a <= b) continue;
          const long nh = open[hi].total - a + b, nl = open[lo].total - b + a;
          if (nh > capacity || nl > capacity) continue;
          const long g = std::labs(nh - nl);
          if (g + min_gain < gap && g < best_gap) { best_gap = g; si = static_cast<int>(i); sj = static_cast<int>(j); }
        }
      }
      if (si < 0) break;
      std::swap(open[hi].lens[si], open[lo].lens[sj]);
      std::swap(open[hi].ids[si], open[lo].ids[sj]);
      open[hi].total = std::accumulate(open[hi].lens.begin(), open[hi].lens.end(), 0L);
      open[lo].total = std::accumulate(open[lo].lens.begin(), open[lo].lens.end(), 0L);
    }
  }

  void start_bucket(long id, long len) {
    Bucket b;
    b.total = len;
    b.ids.push_back(id);
    b.lens.push_back(len);
    open.push_back(std::move(b));
  }

  void add(long id, long len) {
    if (policy == 0) {
      if (!open.empty() && open[0].total > 0 && open[0].total + len > capacity) emit(0);
      if (open.empty()) { start_bucket(id, len); return; }
      open[0].total += len; open[0].ids.push_back(id); open[0].lens.push_back(len);
      return;
    }
    int idx = -1;
    if (policy == 3) {
      for (size_t i = 0; i < open.size(); ++i)
        if (open[i].total + len <= capacity) { idx = static_cast<int>(i); break; }
    } else {
      idx = best_fit(len);
    }
    if (idx >= 0) {
      open[idx].total += len; open[idx].ids.push_back(id); open[idx].lens.push_back(len);
      if ((policy == 1 || policy == 3) && open[idx].total >= fill_full) emit(static_cast<size_t>(idx));
      return;
    }
    if (static_cast<int>(open.size()) < max_open) { start_bucket(id, len); return; }
    if (policy == 2) {
      balance();
      emit(0);  // oldest
      start_bucket(id, len);
    } else {
      size_t fullest = 0;
      for (size_t i = 1; i < open.size(); ++i)
        if (open[i].total > open[fullest].total) fullest = i;
      // keep the slot position of the evicted pack, as a replacement
      ready.push_back(std::move(open[fullest].ids));
      Bucket b;
      b.total = len; b.ids.push_back(id); b.lens.push_back(len);
      open[fullest] = std::move(b);
    }
  }

  void flush() {
    if (policy == 2) balance();
    for (auto& b : open)
      if (!b.ids.empty()) ready.push_back(std::move(b.ids));
    open.clear();
  }
};

}  // namespace

extern "C" {

void* pack_stream_new(int policy, long capacity, int max_open, double fill_threshold, int max_swap_iters,
                      long min_gain) {
  auto* s = new PackStream();
  s->policy = policy;
  s->capacity = capacity;
  s->max_open = policy == 0 ? 1 : std::max(1, max_open);
  s->fill_full = static_cast<long>(static_cast<double>(capacity) * fill_threshold);
  s->max_swap_iters = max_swap_iters;
  s->min_gain = min_gain;
  return s;
}
void pack_stream_free(void* h) { delete static_cast<PackStream*>(h); }
void pack_stream_add(void* h, long id, long len) { static_cast<PackStream*>(h)->add(id, len); }
void pack_stream_flush(void* h) { static_cast<PackStream*>(h)->flush(); }
// number of ready packs; pack_stream_pop copies the oldest into out (capacity cap) and returns its size
int pack_stream_ready(void* h) { return static_cast<int>(static_cast<PackStream*>(h)->ready.size()); }
long pack_stream_pop(void* h, long* out, long cap) {
  auto* s = static_cast<PackStream*>(h);
  if (s->ready.empty()) return -1;
  auto& p = s->ready.front();
  const long n = static_cast<long>(p.size());
  if (n > cap) return -n;
  std::copy(p.begin(), p.end(), out);
  s->ready.erase(s->ready.begin());
  return n;
}

// Offline next-fit over a fixed order: group_of[i] = pack index of sample i.  Samples longer
// than capacity get a pack of their own.  Returns the number of packs.
long offline_first_fit(const long* lens, long n, long capacity, long* group_of) {
  long g = -1, cur = 0;
  for (long i = 0; i < n; ++i) {
    if (g < 0 || cur + lens[i] > capacity) { ++g; cur = 0; }
    group_of[i] = g;
    cur += lens[i];
  }
  return g + 1;
}
// window_N: within consecutive windows of `window` samples, sort by length (descending) and
// first-fit into packs; keeps locality while filling better than next-fit.
long offline_window(const long* lens, long n, long capacity, long window, long* group_of) {
  long next_group = 0;
  std::vector<long> order, totals;
  for (long w0 = 0; w0 < n; w0 += window) {
    const long w1 = std::min(n, w0 + window);
    order.resize(static_cast<size_t>(w1 - w0));
    std::iota(order.begin(), order.end(), w0);
    std::stable_sort(order.begin(), order.end(), [&](long a, long b) { return lens[a] > lens[b]; });
    totals.clear();
    for (long i : order) {
      long placed = -1;
      for (size_t b = 0; b < totals.size(); ++b)
        if (totals[b] + lens[i] <= capacity) { placed = static_cast<long>(b); break; }
      if (placed < 0) { totals.push_back(0); placed = static_cast<long>(totals.size()) - 1; }
      totals[static_cast<size_t>(placed)] += lens[i];
      group_of[i] = next_group + placed;
    }
    next_group += static_cast<long>(totals.size());
  }
  return next_group;
}

// LPT with locality: items (weight w[i], home rank home[i]) sorted by weight descending
// (ties by index) go to the least-loaded rank; among ranks within `slack` of the least
// load the item's home rank is preferred so that data already there does not move.
void lpt_balance(const long* w, const int* home, long n, int ranks, double slack, int* owner, long* load_out) {
  std::vector<long> order(static_cast<size_t>(n));
  std::iota(order.begin(), order.end(), 0L);
  std::stable_sort(order.begin(), order.end(), [&](long a, long b) { return w[a] > w[b]; });
  std::vector<long> load(static_cast<size_t>(ranks), 0);
  for (long i : order) {
    int best = 0;
    for (int r = 1; r < ranks; ++r)
      if (load[r] < load[best]) best = r;
    const int h = home[i];
    if (h >= 0 && h < ranks && h != best) {
      const double lim = static_cast<double>(load[best]) + slack * static_cast<double>(w[i]);
      if (static_cast<double>(load[h]) <= lim) best = h;
    }
    owner[i] = best;
    load[best] += w[i];
  }
  for (int r = 0; r < ranks; ++r) load_out[r] = load[r];
}

}  // extern "C"
