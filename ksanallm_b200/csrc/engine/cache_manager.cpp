#include "cache_manager.h"

#include <algorithm>
#include <string>

namespace ksana {

CacheManager::CacheManager(int num_device_blocks, int num_host_blocks, int block_tokens, bool enable_prefix_cache)
    : block_tokens_(block_tokens), prefix_(enable_prefix_cache), num_host_blocks_(num_host_blocks),
      blocks_(num_device_blocks) {
  free_.reserve(num_device_blocks);
  for (int i = num_device_blocks - 1; i >= 0; --i) free_.push_back(i);   // pop_back hands out 0,1,2,...
  host_free_.reserve(num_host_blocks);
  for (int i = num_host_blocks - 1; i >= 0; --i) host_free_.push_back(i);
}

uint64_t CacheManager::HashTokens(const int* t, int n) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint32_t>(t[i]);
    h *= 0x100000001b3ull;
    h ^= h >> 29;
  }
  return h;
}

uint64_t CacheManager::ChildKey(int parent, uint64_t h) {
  uint64_t x = h ^ (static_cast<uint64_t>(parent + 1) * 0x9E3779B97F4A7C15ull);
  x ^= x >> 31;
  return x * 0xBF58476D1CE4E5B9ull;
}

int CacheManager::FindChild(int parent, const int* t) const {
  const uint64_t key = ChildKey(parent, HashTokens(t, block_tokens_));
  auto it = child_index_.find(key);
  if (it == child_index_.end()) return -1;
  const Block& b = blocks_[it->second];
  if (!b.in_tree || b.parent != parent || !std::equal(b.tokens.begin(), b.tokens.end(), t)) return -1;
  return it->second;
}

int CacheManager::AcquirePrefix(const std::vector<int>& tokens, std::vector<int>* blocks) {
  if (!prefix_) return 0;
  const int full = static_cast<int>(tokens.size()) / block_tokens_;
  int parent = -1, matched = 0;
  for (int i = 0; i < full; ++i) {
    const int id = FindChild(parent, tokens.data() + static_cast<size_t>(i) * block_tokens_);
    if (id < 0) break;
    Block& b = blocks_[id];
    if (b.ref == 0 && b.in_lru) { lru_.erase(b.lru_it); b.in_lru = false; }
    ++b.ref;
    blocks->push_back(id);
    parent = id;
    ++matched;
  }
  if (matched) {
    ++stats_.prefix_hit_requests;
    stats_.prefix_hit_blocks += matched;
    stats_.prefix_hit_tokens += static_cast<int64_t>(matched) * block_tokens_;
  }
  return matched * block_tokens_;
}

void CacheManager::RemoveFromTree(int id) {
  Block& b = blocks_[id];
  if (!b.in_tree) return;
  child_index_.erase(b.key);
  auto range = content_index_.equal_range(b.content_hash);
  for (auto it = range.first; it != range.second; ++it) {
    if (it->second == id) { content_index_.erase(it); break; }
  }
  if (b.parent >= 0) {
    auto& sib = blocks_[b.parent].children;
    sib.erase(std::remove(sib.begin(), sib.end(), id), sib.end());
  }
  if (b.in_lru) { lru_.erase(b.lru_it); b.in_lru = false; }
  b.in_tree = false;
  b.parent = -1;
  b.tokens.clear();
}

void CacheManager::EvictSubtree(int id) {
  // iterative post-order: children first
  std::vector<int> stack{id}, order;
  while (!stack.empty()) {
    const int cur = stack.back();
    stack.pop_back();
    order.push_back(cur);
    for (int c : blocks_[cur].children) stack.push_back(c);
  }
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    Block& b = blocks_[*it];
    b.children.clear();
    RemoveFromTree(*it);
    if (b.ref == 0) {            // by construction descendants of an unreferenced node are unreferenced
      free_.push_back(*it);
      ++stats_.evicted_blocks;
    }
  }
}

bool CacheManager::EnsureFree(int n) {
  if (usable_blocks() < n) return false;
  while (static_cast<int>(free_.size()) < n && !lru_.empty()) EvictSubtree(lru_.front());
  return static_cast<int>(free_.size()) >= n;
}

bool CacheManager::Allocate(int n, std::vector<int>* blocks) {
  if (n <= 0) return true;
  if (!EnsureFree(n)) return false;
  for (int i = 0; i < n; ++i) {
    const int id = free_.back();
    free_.pop_back();
    blocks_[id].ref = 1;
    blocks->push_back(id);
  }
  return true;
}

void CacheManager::Release(const std::vector<int>& ids) {
  // leaf-most first so that a chain released together ages leaf-first in the LRU order
  for (auto it = ids.rbegin(); it != ids.rend(); ++it) {
    Block& b = blocks_[*it];
    if (b.ref <= 0) continue;
    if (--b.ref > 0) continue;
    if (b.in_tree) {
      lru_.push_back(*it);
      b.lru_it = std::prev(lru_.end());
      b.in_lru = true;
    } else {
      free_.push_back(*it);
    }
  }
}

int CacheManager::Promote(const std::vector<int>& tokens, std::vector<int>* blocks, int computed_tokens,
                          int first_unpromoted) {
  if (!prefix_) return first_unpromoted;
  const int full = std::min(computed_tokens / block_tokens_, static_cast<int>(blocks->size()));
  int i = first_unpromoted;
  for (; i < full; ++i) {
    const int parent = i == 0 ? -1 : (*blocks)[i - 1];
    if (parent >= 0 && !blocks_[parent].in_tree) break;
    const int own = (*blocks)[i];
    if (blocks_[own].in_tree) continue;     // reached through a prefix hit
    const int* t = tokens.data() + static_cast<size_t>(i) * block_tokens_;
    const int existing = FindChild(parent, t);
    if (existing >= 0 && existing != own) {
      Block& e = blocks_[existing];
      if (e.ref == 0 && e.in_lru) { lru_.erase(e.lru_it); e.in_lru = false; }
      ++e.ref;
      (*blocks)[i] = existing;
      Release({own});
      ++stats_.dedup_blocks;
      continue;
    }
    Block& b = blocks_[own];
    if (b.ref != 1) break;   // a block shared by forked siblings is promoted by whichever fills it first
    b.in_tree = true;
    b.parent = parent;
    b.tokens.assign(t, t + block_tokens_);
    b.content_hash = HashTokens(t, block_tokens_);
    b.key = ChildKey(parent, b.content_hash);
    child_index_[b.key] = own;
    content_index_.emplace(b.content_hash, own);
    if (parent >= 0) blocks_[parent].children.push_back(own);
  }
  return i;
}

bool CacheManager::Fork(const std::vector<int>& src_blocks, int cached_tokens, std::vector<int>* dst_blocks,
                        std::vector<BlockCopy>* copies) {
  const int full = cached_tokens / block_tokens_;
  const bool tail = cached_tokens % block_tokens_ != 0 && full < static_cast<int>(src_blocks.size());
  std::vector<int> fresh;
  if (tail && !Allocate(1, &fresh)) return false;
  for (int i = 0; i < full && i < static_cast<int>(src_blocks.size()); ++i) {
    ++blocks_[src_blocks[i]].ref;
    dst_blocks->push_back(src_blocks[i]);
  }
  if (tail) {
    dst_blocks->push_back(fresh[0]);
    copies->push_back({src_blocks[full], fresh[0], 0});
  }
  return true;
}

bool CacheManager::SwapOut(std::vector<int>* blocks, std::vector<int>* host_blocks, std::vector<SwapCopy>* copies) {
  int keep = static_cast<int>(blocks->size());
  while (keep > 0 && blocks_[(*blocks)[keep - 1]].ref == 1) --keep;
  const int n = static_cast<int>(blocks->size()) - keep;
  if (n == 0) return true;
  if (static_cast<int>(host_free_.size()) < n) return false;
  for (int i = keep; i < static_cast<int>(blocks->size()); ++i) {
    const int id = (*blocks)[i];
    Block& b = blocks_[id];
    if (b.in_tree) {
      // unreferenced cached descendants cannot outlive their parent
      while (!b.children.empty()) EvictSubtree(b.children.back());
      RemoveFromTree(id);
    }
    const int h = host_free_.back();
    host_free_.pop_back();
    host_blocks->push_back(h);
    copies->push_back({id, h});
    b.ref = 0;
    free_.push_back(id);
    ++stats_.swapped_out_blocks;
  }
  blocks->resize(keep);
  return true;
}

bool CacheManager::SwapIn(std::vector<int>* blocks, std::vector<int>* host_blocks, std::vector<SwapCopy>* copies) {
  const int n = static_cast<int>(host_blocks->size());
  std::vector<int> fresh;
  if (!Allocate(n, &fresh)) return false;
  for (int i = 0; i < n; ++i) {
    copies->push_back({fresh[i], (*host_blocks)[i]});
    blocks->push_back(fresh[i]);
    host_free_.push_back((*host_blocks)[i]);
    ++stats_.swapped_in_blocks;
  }
  host_blocks->clear();
  return true;
}

void CacheManager::ReleaseHost(const std::vector<int>& host_blocks) {
  for (int h : host_blocks) host_free_.push_back(h);
}

int CacheManager::AcquireFlexible(const std::vector<int>& tokens, int prefix_tokens, int min_tokens,
                                  std::vector<int>* blocks, std::vector<BlockCopy>* copies) {
  if (!prefix_ || min_tokens <= 0) return 0;
  const int B = block_tokens_;
  const int first = prefix_tokens / B;
  // leave at least one token to compute
  const int last = (static_cast<int>(tokens.size()) - 1) / B;
  std::vector<std::pair<int, int>> run;   // (source block, position delta in tokens)
  for (int i = first; i < last; ++i) {
    const int* t = tokens.data() + static_cast<size_t>(i) * B;
    const uint64_t h = HashTokens(t, B);
    int src = -1;
    auto range = content_index_.equal_range(h);
    for (auto it = range.first; it != range.second; ++it) {
      const Block& c = blocks_[it->second];
      if (c.in_tree && std::equal(c.tokens.begin(), c.tokens.end(), t)) { src = it->second; break; }
    }
    if (src < 0) break;
    int depth = 0;   // source position = depth of the node in the tree
    for (int p = blocks_[src].parent; p >= 0; p = blocks_[p].parent) ++depth;
    run.emplace_back(src, (i - depth) * B);
  }
  if (static_cast<int>(run.size()) * B < min_tokens) return 0;
  // pin the sources while allocating so that eviction cannot take them
  std::vector<int> pinned;
  for (auto& r : run) {
    Block& b = blocks_[r.first];
    if (b.ref == 0 && b.in_lru) { lru_.erase(b.lru_it); b.in_lru = false; }
    ++b.ref;
    pinned.push_back(r.first);
  }
  std::vector<int> fresh;
  const bool ok = Allocate(static_cast<int>(run.size()), &fresh);
  if (ok) {
    for (size_t i = 0; i < run.size(); ++i) {
      blocks->push_back(fresh[i]);
      copies->push_back({run[i].first, fresh[i], run[i].second});
    }
    stats_.flexible_hit_tokens += static_cast<int64_t>(run.size()) * B;
  }
  Release(pinned);
  return ok ? static_cast<int>(run.size()) * B : 0;
}

bool CacheManager::CheckInvariants(std::string* why) const {
  std::vector<int> state(blocks_.size(), 0);
  for (int id : free_) {
    if (state[id]++) { *why = "block twice in free list"; return false; }
    if (blocks_[id].ref != 0 || blocks_[id].in_tree) { *why = "free block referenced or cached"; return false; }
  }
  for (int id : lru_) {
    if (state[id]++) { *why = "evictable block also free"; return false; }
    if (blocks_[id].ref != 0 || !blocks_[id].in_tree) { *why = "evictable block referenced or not cached"; return false; }
  }
  for (size_t id = 0; id < blocks_.size(); ++id) {
    if (!state[id] && blocks_[id].ref <= 0) { *why = "leaked block " + std::to_string(id); return false; }
    if (blocks_[id].in_tree && blocks_[id].parent >= 0 && !blocks_[blocks_[id].parent].in_tree) {
      *why = "cached block with uncached parent";
      return false;
    }
  }
  return true;
}

}  // namespace ksana
