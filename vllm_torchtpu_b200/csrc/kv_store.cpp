// Host-side index of the KV offload store: which content hash lives in which slot of the pinned
// slab, with LRU eviction and pin counts for slots that have a transfer in flight.
//
// The slab itself (pinned, device-mapped host memory laid out [layer][slot][block_bytes]) is
// allocated by the caller; this index only hands out slot numbers, so the GPU block-copy kernel
// can move blocks between the paged pool and the slab by slot id.  Thread safe.
//
// Plays the role of the reference's native KVCacheStore behind its offloading connector
// (reference: src/vllm_torchtpu/offload/raiden_store.py:227-2722).
#include <cstdint>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Slot {
  uint64_t key = 0;
  bool used = false;
  bool committed = false;
  int pins = 0;
  std::list<int>::iterator lru_it;
};

struct Store {
  std::mutex mu;
  std::vector<Slot> slots;
  std::unordered_map<uint64_t, int> index;
  std::list<int> lru;            // front = coldest
  std::vector<int> free_list;
  uint64_t hits = 0, misses = 0, evictions = 0;
};

}  // namespace

extern "C" {

void* b200_store_create(int capacity) {
  auto* s = new Store();
  s->slots.resize(capacity);
  for (int i = capacity - 1; i >= 0; --i) s->free_list.push_back(i);
  return s;
}

void b200_store_destroy(void* h) { delete static_cast<Store*>(h); }

// Longest prefix of keys[0..n) that is committed; pins the hit slots and writes them to slots_out.
int b200_store_lookup_prefix(void* h, const uint64_t* keys, int n, int* slots_out, int pin) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  int i = 0;
  for (; i < n; ++i) {
    auto it = s->index.find(keys[i]);
    if (it == s->index.end() || !s->slots[it->second].committed) break;
    Slot& sl = s->slots[it->second];
    slots_out[i] = it->second;
    if (pin) ++sl.pins;
    s->lru.erase(sl.lru_it);
    s->lru.push_back(it->second);
    sl.lru_it = std::prev(s->lru.end());
  }
  s->hits += i;
  s->misses += (n - i);
  return i;
}

// Reserve a slot for `key` (evicting the coldest unpinned slot when full).  Returns the slot,
// -1 when everything is pinned, or -2-slot when the key is already stored (nothing to do).
int b200_store_reserve(void* h, uint64_t key) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  auto it = s->index.find(key);
  if (it != s->index.end()) return -2 - it->second;
  int slot = -1;
  if (!s->free_list.empty()) {
    slot = s->free_list.back();
    s->free_list.pop_back();
  } else {
    for (auto li = s->lru.begin(); li != s->lru.end(); ++li) {
      if (s->slots[*li].pins == 0) {
        slot = *li;
        s->index.erase(s->slots[slot].key);
        s->lru.erase(li);
        ++s->evictions;
        break;
      }
    }
  }
  if (slot < 0) return -1;
  Slot& sl = s->slots[slot];
  sl.key = key;
  sl.used = true;
  sl.committed = false;
  sl.pins = 1;                       // pinned until commit
  s->index[key] = slot;
  s->lru.push_back(slot);
  sl.lru_it = std::prev(s->lru.end());
  return slot;
}

// The data of a reserved slot has landed (ok = 1) or the save failed (ok = 0: slot is released).
void b200_store_commit(void* h, int slot, int ok) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  Slot& sl = s->slots[slot];
  if (sl.pins > 0) --sl.pins;
  if (ok) {
    sl.committed = true;
  } else {
    s->index.erase(sl.key);
    s->lru.erase(sl.lru_it);
    sl.used = false;
    s->free_list.push_back(slot);
  }
}

void b200_store_unpin(void* h, const int* slots, int n) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  for (int i = 0; i < n; ++i)
    if (s->slots[slots[i]].pins > 0) --s->slots[slots[i]].pins;
}

// Sum of the pin counts of all slots (slots with a lookup or a save in flight).
int b200_store_pinned(void* h) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  int n = 0;
  for (const Slot& sl : s->slots) n += sl.pins;
  return n;
}

void b200_store_stats(void* h, uint64_t* out4) {
  auto* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lock(s->mu);
  out4[0] = s->hits;
  out4[1] = s->misses;
  out4[2] = s->evictions;
  out4[3] = s->index.size();
}

}  // extern "C"
