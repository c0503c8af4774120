// Karmarkar-Karp (largest differencing method) k-way partitioning of sequence workloads, used by the
// Data Coordinator to balance tokens across data-parallel ranks and across micro-batches.
// Same contract as the reference's Python implementation (siirl/utils/model_utils/seqlen_balancing.py:41-142):
// items are merged through a max-heap of partial partitions keyed by the spread between their heaviest and
// lightest set; with equal_size every set receives the same number of items (n must divide by k).
#include <algorithm>
#include <cstdint>
#include <queue>
#include <vector>

namespace {

struct Set {
  long long sum = 0;
  std::vector<int> items;
};

struct State {
  std::vector<Set> sets;  // kept sorted by (sum, size) descending
  long long spread() const { return sets.front().sum - sets.back().sum; }
  void sort_sets() {
    std::sort(sets.begin(), sets.end(), [](const Set& a, const Set& b) {
      if (a.sum != b.sum) return a.sum > b.sum;
      return a.items.size() > b.items.size();
    });
  }
};

struct Cmp {
  bool operator()(const State* a, const State* b) const {
    if (a->spread() != b->spread()) return a->spread() < b->spread();
    return a->sets.front().sum < b->sets.front().sum;
  }
};

}  // namespace

extern "C" int sb_kk_partition(const long long* workloads, int n, int k, int equal_size, int* out_part) {
  if (k <= 0 || n < 0) return -3;
  if (equal_size && n % k != 0) return -3;
  std::vector<std::pair<long long, int>> order(n);
  for (int i = 0; i < n; ++i) order[i] = {workloads[i], i};
  std::sort(order.begin(), order.end());
  std::vector<State*> owned;
  std::priority_queue<State*, std::vector<State*>, Cmp> heap;
  if (equal_size) {
    for (int off = 0; off < n; off += k) {
      State* s = new State();
      s->sets.resize(k);
      for (int j = 0; j < k; ++j) {
        s->sets[j].sum = order[off + j].first;
        s->sets[j].items.push_back(order[off + j].second);
      }
      s->sort_sets();
      owned.push_back(s);
      heap.push(s);
    }
  } else {
    for (int i = 0; i < n; ++i) {
      State* s = new State();
      s->sets.resize(k);
      s->sets[0].sum = order[i].first;
      s->sets[0].items.push_back(order[i].second);
      s->sort_sets();
      owned.push_back(s);
      heap.push(s);
    }
  }
  if (heap.empty()) return 0;
  while (heap.size() > 1) {
    State* a = heap.top();
    heap.pop();
    State* b = heap.top();
    heap.pop();
    // pair the heaviest sets of one with the lightest sets of the other
    for (int j = 0; j < k; ++j) {
      Set& dst = a->sets[j];
      Set& src = b->sets[k - 1 - j];
      dst.sum += src.sum;
      dst.items.insert(dst.items.end(), src.items.begin(), src.items.end());
    }
    a->sort_sets();
    heap.push(a);
  }
  State* fin = heap.top();
  for (int j = 0; j < k; ++j)
    for (int it : fin->sets[j].items) out_part[it] = j;
  for (State* s : owned) delete s;
  return 0;
}
