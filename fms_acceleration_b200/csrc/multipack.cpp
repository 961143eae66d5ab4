// Host-side multipack batch allocator (C++), the compiled counterpart of the numba-jitted allocator the
// reference uses (fms_acceleration_aadp/multipack_sampler.py:230-395).
//
// Problem: samples with token lengths len[0..count) arrive in a fixed (already shuffled) order.  Cut the
// sequence into consecutive runs; each run is distributed over `n` ranks ("bins") so that every bin holds at
// most `c` tokens (or, with padding, max_len_in_bin * samples_in_bin <= c).  Runs are made as long as
// possible: the run length is found by binary search on "does first-fit-decreasing pack this prefix into n
// bins", bounded above by the number of samples whose total length is <= c * n.  Allocation stops at the
// first run that no longer fills all n bins.  The caller's rank receives its bin of every run.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

namespace {

struct Packer {
  int64_t c;
  int n;
  bool padding;
  std::vector<int64_t> sorted;
  std::vector<int64_t> free_or_max;  // no padding: remaining capacity; padding: longest sample in the bin
  std::vector<int64_t> counts;

  // can len[0..m) be packed into at most n bins?
  bool fits(const int64_t* len, int64_t m) {
    sorted.assign(len, len + m);
    std::sort(sorted.begin(), sorted.end(), std::greater<int64_t>());
    if (!padding) {
      free_or_max.assign(n, c);
      for (int64_t s : sorted) {
        bool placed = false;
        for (int b = 0; b < n; ++b) {
          if (free_or_max[b] >= s) {
            free_or_max[b] -= s;
            placed = true;
            break;
          }
        }
        if (!placed) return false;
      }
      return true;
    }
    free_or_max.assign(n, 0);
    counts.assign(n, 0);
    for (int64_t s : sorted) {
      bool placed = false;
      for (int b = 0; b < n; ++b) {
        const int64_t longest = std::max(free_or_max[b], s);
        if (longest * (counts[b] + 1) <= c) {
          free_or_max[b] = longest;
          counts[b] += 1;
          placed = true;
          break;
        }
      }
      if (!placed) return false;
    }
    return true;
  }

  // first-fit-decreasing with the assignment returned; bins open on demand
  void assign(const int64_t* len, int64_t m, int64_t start, std::vector<std::vector<int64_t>>& bins) {
    std::vector<int64_t> order(m);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return len[a] > len[b]; });
    bins.clear();
    std::vector<int64_t> state, cnt;
    for (int64_t i : order) {
      const int64_t s = len[i];
      bool placed = false;
      for (size_t b = 0; b < bins.size(); ++b) {
        if (!padding) {
          if (state[b] >= s) {
            state[b] -= s;
            bins[b].push_back(start + i);
            placed = true;
            break;
          }
        } else {
          const int64_t longest = std::max(state[b], s);
          if (longest * (cnt[b] + 1) <= c) {
            state[b] = longest;
            cnt[b] += 1;
            bins[b].push_back(start + i);
            placed = true;
            break;
          }
        }
      }
      if (!placed) {
        bins.emplace_back(1, start + i);
        state.push_back(padding ? s : c - s);
        cnt.push_back(1);
      }
    }
  }
};

}  // namespace

// out_idx   : capacity `count`; sample positions (into `lengths`) of this rank's batches, concatenated
// out_off   : capacity `count + 1`; batch b is out_idx[out_off[b] .. out_off[b+1])
// stats[0]  : number of batches; stats[1]: tokens consumed by all ranks; stats[2]: token slots offered
extern "C" int fmsb_multipack_allocate(const int64_t* lengths, int64_t count, int rank, int64_t c, int n, int padding,
                                       int64_t* out_idx, int64_t* out_off, int64_t* stats) {
  if (n <= 0 || rank < 0 || rank >= n || c <= 0) return -2;
  std::vector<int64_t> cumsum(count);
  int64_t acc = 0;
  for (int64_t i = 0; i < count; ++i) {
    acc += lengths[i];
    cumsum[i] = acc;
  }
  Packer pk{c, n, padding != 0, {}, {}, {}};
  std::vector<std::vector<int64_t>> bins;
  int64_t start = 0, consumed = 0, nb = 0, written = 0;
  out_off[0] = 0;
  while (true) {
    // samples from `start` whose running total stays within c * n
    const int64_t limit = consumed + c * (int64_t)n;
    const int64_t upto = std::upper_bound(cumsum.begin() + start, cumsum.end(), limit) - (cumsum.begin() + start);
    int64_t lo = 1, hi = 1 + upto;
    while (hi - lo > 1) {
      const int64_t mid = (lo + hi) / 2;
      if (pk.fits(lengths + start, mid)) lo = mid; else hi = mid;
    }
    const int64_t take = std::min<int64_t>(lo, count - start);
    pk.assign(lengths + start, take, start, bins);
    if ((int)bins.size() < n) break;
    if ((int)bins.size() > n) return -3;  // cannot happen when every sample fits in one bin
    start += take;
    consumed = cumsum[start - 1];
    for (int64_t v : bins[rank]) out_idx[written++] = v;
    out_off[++nb] = written;
  }
  stats[0] = nb;
  stats[1] = consumed;
  stats[2] = nb * c * (int64_t)n;
  return 0;
}
