// Host-side planners: tensor-parallel slices, MoE residency ranking, per-step expert dispatch tiers, slot book.
//
// Reference counterparts: cpp_runtime/core/include/mfq/tensor_parallel.h:23-140 (weighted, granularity-aligned
// contiguous slices), moe_residency_ranker.h:13-67 (heat-based swap pairs), moe_dispatch_plan.h:10-162 (CPU /
// GPU-resident / GPU-transfer / inactive with a measured cost model), engine/include/moe_cache_policy.h (slot book LRU).
#include "common.h"
#include "mfq_core.h"

#include <list>
#include <numeric>
#include <unordered_map>

using mfqn::fail;

extern "C" {

int mfq_tp_plan(int64_t total, int ranks, const double* weights, int64_t granularity, int64_t* begin_out, int64_t* end_out) {
  if (ranks < 1 || granularity < 1 || total < 0 || total % granularity) return fail(-1, "total must be a multiple of the granularity");
  const int64_t units = total / granularity;
  double sum = 0;
  for (int r = 0; r < ranks; ++r) {
    const double w = weights ? weights[r] : 1.0;
    if (!(w >= 0)) return fail(-1, "weights must be non-negative");
    sum += w;
  }
  if (sum <= 0) return fail(-1, "at least one rank needs a positive weight");
  // largest-remainder apportionment of whole units, then contiguous placement in rank order
  std::vector<int64_t> share(ranks);
  std::vector<std::pair<double, int>> rem(ranks);
  int64_t given = 0;
  for (int r = 0; r < ranks; ++r) {
    const double exact = double(units) * (weights ? weights[r] : 1.0) / sum;
    share[r] = int64_t(exact);
    rem[r] = {exact - double(share[r]), r};
    given += share[r];
  }
  std::stable_sort(rem.begin(), rem.end(), [](auto& a, auto& b) { return a.first > b.first; });
  for (int i = 0; given < units; ++i, ++given) ++share[rem[i % ranks].second];
  int64_t at = 0;
  for (int r = 0; r < ranks; ++r) {
    begin_out[r] = at * granularity;
    at += share[r];
    end_out[r] = at * granularity;
  }
  return 0;
}

int mfq_moe_rank_swaps(const double* heat, const uint8_t* resident, int n, int max_swaps, double hysteresis, int* evict_out, int* load_out) {
  if (n <= 0 || max_swaps < 0) return fail(-1, "bad arguments");
  std::vector<int> in, out;
  for (int e = 0; e < n; ++e) (resident[e] ? in : out).push_back(e);
  std::stable_sort(in.begin(), in.end(), [&](int a, int b) { return heat[a] < heat[b]; });    // coldest resident first
  std::stable_sort(out.begin(), out.end(), [&](int a, int b) { return heat[a] > heat[b]; });  // hottest absent first
  int swaps = 0;
  for (size_t i = 0; i < in.size() && i < out.size() && swaps < max_swaps; ++i) {
    // a swap has to pay for its transfer: the newcomer must be hotter by the hysteresis margin
    if (heat[out[i]] <= heat[in[i]] * (1.0 + hysteresis) + 1e-12) break;
    evict_out[swaps] = in[i];
    load_out[swaps] = out[i];
    ++swaps;
  }
  return swaps;
}

int mfq_moe_dispatch_plan(const int* tokens, const uint8_t* resident, int n, double bytes_per_expert, double h2d_gbs,
                          double gpu_tok_us, double cpu_tok_us, int cpu_available, int* tier_out) {
  if (n <= 0 || h2d_gbs <= 0) return fail(-1, "bad arguments");
  const double transfer_us = bytes_per_expert / (h2d_gbs * 1e3);  // GB/s = 1e3 bytes/us
  for (int e = 0; e < n; ++e) {
    if (tokens[e] <= 0) { tier_out[e] = 0; continue; }
    if (resident[e]) { tier_out[e] = 1; continue; }
    const double gpu_cost = transfer_us + gpu_tok_us * tokens[e];
    const double cpu_cost = cpu_tok_us * tokens[e];
    tier_out[e] = (cpu_available && cpu_cost < gpu_cost) ? 3 : 2;
  }
  return 0;
}

namespace {
struct SlotBook {
  struct Item { int64_t key; int slot; int pins; };
  std::list<Item> lru;  // most recent at the back
  std::unordered_map<int64_t, std::list<Item>::iterator> index;
  std::vector<int> free_slots;
};
}  // namespace

void* mfq_slotbook_open(int slots) {
  if (slots <= 0) { fail(-1, "slot count must be positive"); return nullptr; }
  auto* b = new SlotBook();
  for (int s = slots - 1; s >= 0; --s) b->free_slots.push_back(s);
  return b;
}

void mfq_slotbook_close(void* book) { delete static_cast<SlotBook*>(book); }

int mfq_slotbook_lookup(void* book, int64_t key) {
  auto* b = static_cast<SlotBook*>(book);
  auto it = b->index.find(key);
  if (it == b->index.end()) return -1;
  b->lru.splice(b->lru.end(), b->lru, it->second);
  return it->second->slot;
}

int mfq_slotbook_acquire(void* book, int64_t key, int64_t* evicted_key) {
  auto* b = static_cast<SlotBook*>(book);
  if (evicted_key) *evicted_key = -1;
  const int hit = mfq_slotbook_lookup(book, key);
  if (hit >= 0) return hit;
  int slot = -1;
  if (!b->free_slots.empty()) {
    slot = b->free_slots.back();
    b->free_slots.pop_back();
  } else {
    for (auto it = b->lru.begin(); it != b->lru.end(); ++it) {
      if (it->pins > 0) continue;
      slot = it->slot;
      if (evicted_key) *evicted_key = it->key;
      b->index.erase(it->key);
      b->lru.erase(it);
      break;
    }
    if (slot < 0) return fail(-2, "every slot is pinned");
  }
  b->lru.push_back({key, slot, 0});
  b->index[key] = std::prev(b->lru.end());
  return slot;
}

int mfq_slotbook_pin(void* book, int64_t key, int delta) {
  auto* b = static_cast<SlotBook*>(book);
  auto it = b->index.find(key);
  if (it == b->index.end()) return fail(-1, "key not in the book");
  it->second->pins = std::max(0, it->second->pins + delta);
  return it->second->pins;
}
}
