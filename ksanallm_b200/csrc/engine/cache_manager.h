// Paged KV-cache bookkeeping: a pool of device blocks, a pool of pinned-host blocks, and (when
// prefix caching is on) a radix tree over full blocks of token ids.
//
// Design points:
//  * Every block is reference counted. A full block is immutable, so it can be shared by any
//    number of sequences: prefix hits, parallel-sampling siblings and beam forks all share by
//    reference; only a partially filled tail block is ever copied (copy-on-write), instead of
//    the device-to-device copies of whole histories a beam fork costs in the reference
//    (src/ksana_llm/samplers/beam_search/beam_search_sampling.cpp:10-43).
//  * A block id is valid on every tensor-parallel rank: ranks allocate identical pools and
//    follow the scheduler's decisions in lock step, so one id names the per-rank blocks.
//  * Swap and copy operations are returned as lists; the runtime executes them with one gather /
//    scatter kernel on the compute stream ahead of the forward pass, so a block released by a
//    swap-out can be reused in the same step without any asynchronous pending state.
//
// Behavioural counterpart of src/ksana_llm/cache_manager/prefix_cache_manager.cpp:34-1105,
// direct_cache_manager.cpp:17-371 and src/ksana_llm/block_manager/block_manager.cpp:23-301.
#pragma once
#include <cstdint>
#include <list>
#include <string>
#include <unordered_map>
#include <vector>

namespace ksana {

struct BlockCopy { int src; int dst; int pos_delta; };   // device -> device (pos_delta: RoPE re-rotation for flexible cache)
struct SwapCopy { int device_block; int host_block; };

struct CacheStats {
  int64_t prefix_hit_requests = 0, prefix_hit_tokens = 0, prefix_hit_blocks = 0;
  int64_t evicted_blocks = 0, swapped_out_blocks = 0, swapped_in_blocks = 0, dedup_blocks = 0;
  int64_t flexible_hit_tokens = 0;
  CacheStats& operator+=(const CacheStats& o) {
    prefix_hit_requests += o.prefix_hit_requests; prefix_hit_tokens += o.prefix_hit_tokens;
    prefix_hit_blocks += o.prefix_hit_blocks; evicted_blocks += o.evicted_blocks;
    swapped_out_blocks += o.swapped_out_blocks; swapped_in_blocks += o.swapped_in_blocks;
    dedup_blocks += o.dedup_blocks; flexible_hit_tokens += o.flexible_hit_tokens;
    return *this;
  }
};

class CacheManager {
 public:
  CacheManager(int num_device_blocks, int num_host_blocks, int block_tokens, bool enable_prefix_cache);

  int block_tokens() const { return block_tokens_; }
  int num_device_blocks() const { return static_cast<int>(blocks_.size()); }
  int num_host_blocks() const { return num_host_blocks_; }
  int free_blocks() const { return static_cast<int>(free_.size()); }
  int evictable_blocks() const { return static_cast<int>(lru_.size()); }
  int usable_blocks() const { return free_blocks() + evictable_blocks(); }
  int used_blocks() const { return num_device_blocks() - usable_blocks(); }
  int free_host_blocks() const { return static_cast<int>(host_free_.size()); }
  bool prefix_enabled() const { return prefix_; }
  const CacheStats& stats() const { return stats_; }
  int ref_count(int id) const { return blocks_[id].ref; }
  bool in_tree(int id) const { return blocks_[id].in_tree; }

  // Longest cached prefix of `tokens` in whole blocks. Takes one reference on each matched block
  // and appends it to `blocks` (which must be empty). Returns the matched token count.
  int AcquirePrefix(const std::vector<int>& tokens, std::vector<int>* blocks);

  // n fresh private blocks (ref 1), evicting least-recently-released cached blocks when the free
  // list runs short. All-or-nothing.
  bool Allocate(int n, std::vector<int>* blocks);

  // Drop one reference on each block. Cached blocks nobody references become evictable (and stay
  // matchable); private ones return to the free list.
  void Release(const std::vector<int>& blocks);

  // Enter the sequence's newly filled blocks [first_unpromoted, computed_tokens / B) into the tree.
  // If an identical block is already cached the sequence is re-pointed to it and its own copy is
  // freed. Returns the new count of promoted blocks.
  int Promote(const std::vector<int>& tokens, std::vector<int>* blocks, int computed_tokens, int first_unpromoted);

  // Share `src` history with a new sequence: full blocks by reference, the partial tail (if any)
  // through a fresh block plus a copy task.
  bool Fork(const std::vector<int>& src_blocks, int cached_tokens, std::vector<int>* dst_blocks,
            std::vector<BlockCopy>* copies);

  // Move the sequence's exclusively owned tail blocks to host memory. `blocks` keeps the shared
  // head; the swapped tail is described by `host_blocks`. False (nothing changed) when the host
  // pool cannot take the tail.
  bool SwapOut(std::vector<int>* blocks, std::vector<int>* host_blocks, std::vector<SwapCopy>* copies);
  // Bring a swapped tail back (all-or-nothing); the caller re-promotes afterwards.
  bool SwapIn(std::vector<int>* blocks, std::vector<int>* host_blocks, std::vector<SwapCopy>* copies);
  void ReleaseHost(const std::vector<int>& host_blocks);

  // Non-prefix reuse ("flexible cache"): after the matched prefix, look for cached blocks whose
  // token content equals the next block-aligned windows of `tokens` although they sit at another
  // position; needs at least `min_tokens` consecutive tokens. Allocates destination blocks into
  // `blocks` and emits copy tasks carrying the position delta for RoPE re-rotation.
  int AcquireFlexible(const std::vector<int>& tokens, int prefix_tokens, int min_tokens, std::vector<int>* blocks,
                      std::vector<BlockCopy>* copies);

  // Consistency check used by tests: every block is in exactly one of {free, evictable, referenced}.
  bool CheckInvariants(std::string* why) const;

 private:
  struct Block {
    int ref = 0;
    bool in_tree = false;
    bool in_lru = false;
    int parent = -1;
    uint64_t key = 0;
    uint64_t content_hash = 0;
    std::vector<int> tokens;
    std::vector<int> children;
    std::list<int>::iterator lru_it;
  };
  static uint64_t HashTokens(const int* t, int n);
  static uint64_t ChildKey(int parent, uint64_t h);
  int FindChild(int parent, const int* t) const;
  void RemoveFromTree(int id);          // detaches one node (children must be gone)
  void EvictSubtree(int id);            // frees an unreferenced node with all its descendants
  bool EnsureFree(int n);

  int block_tokens_;
  bool prefix_;
  int num_host_blocks_;
  std::vector<Block> blocks_;
  std::vector<int> free_;
  std::vector<int> host_free_;
  std::list<int> lru_;                  // evictable cached blocks, oldest first
  std::unordered_map<uint64_t, int> child_index_;
  std::unordered_multimap<uint64_t, int> content_index_;   // block content -> cached blocks (flexible cache)
  CacheStats stats_;
};

}  // namespace ksana
