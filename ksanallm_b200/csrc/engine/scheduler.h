// Continuous-batching scheduler: owns the sequences and their KV blocks and turns the request
// queues into one StepPlan per engine step.
//
// The per-step passes and thresholds follow the reference strategy
// (src/ksana_llm/batch_scheduler/strategy/continuous_batching.cpp:28-841,
//  src/ksana_llm/batch_scheduler/batch_scheduler.cpp:53-158): admission limits, waiting timeout,
// abort, running -> swapped -> waiting priority, swap-out / swap-in / launch block thresholds,
// SWAP or RECOMPUTE preemption of the most recently admitted request, split-fuse chunked prefill.
// Differences that come from the block design (see cache_manager.h): swaps are executed on the
// compute stream at the start of the step that decided them, so there are no pending-swap queues;
// sibling sequences (parallel sampling, beams) fork from one prefill instead of each running its own.
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.h"
#include "common.h"

namespace ksana {

struct SchedulerConfig {
  int schedule_strategy = 0;            // 0 continuous batching, 1 auto (static) batching
  int64_t waiting_timeout_in_ms = 600000;
  int max_waiting_queue_len = 256;
  int max_step_tokens = 4096;
  int max_batch_size = 8;
  int max_token_len = 2048;
  float swapout_block_threshold = 1.0f;
  float swapin_block_threshold = 2.0f;
  float launch_block_threshold = 2.0f;
  int preempt_mode = 0;                 // 0 SWAP, 1 RECOMPUTE
  int split_fuse_token_num = 0;
  int min_flexible_cache_num = 0;
  bool enable_prefix_cache = false;
  int block_token_num = 16;
  int auto_batch_wait_ms = 100;
  // attention data parallelism: sequence s lives on rank s % dp_size and only that rank holds its KV blocks, so
  // every rank gets a block pool (and prefix tree, and host swap pool) of its own; block ids are per rank
  int dp_size = 1;
  std::vector<int> eos_token_ids;
};

enum class SeqState : int { WAITING = 0, RUNNING = 1, SWAPPED = 2, FINISHED = 3 };

struct Sequence {
  int64_t seq_id = 0;
  int64_t req_id = 0;
  int index = 0;                 // position inside its request group
  std::vector<int> tokens;       // prompt + generated
  int prompt_len = 0;
  int kv_cached = 0;             // tokens whose K/V is in the cache
  int chunk = 0;                 // tokens forwarded in the step being planned / executed
  int promoted = 0;              // blocks entered into the prefix tree
  int prefix_hit_tokens = 0;
  int flexible_hit_tokens = 0;
  int sampled = 0;               // tokens sampled so far (RNG counter)
  std::vector<int> blocks;
  std::vector<int> host_blocks;
  std::shared_ptr<SamplingConfig> cfg;
  int64_t arrive_ms = 0;
  int64_t first_token_ms = 0;
  bool aborted = false;
  // Pipelined stepping (see Scheduler::Advance / Resolve): the last element of `tokens` is a placeholder (-1) for a
  // token that was sampled on the device by a step whose results the host has not read yet; `draining`: that token
  // is certainly the sequence's last one (length limits), so it is not scheduled again while it is outstanding
  bool token_pending = false;
  bool draining = false;
  bool forked_pending = false;   // sibling that waits for its leader's prefill
  int64_t leader = -1;
  SeqState state = SeqState::WAITING;
  Status finish_status;
  int preempt_count = 0;
};

struct SeqEvent {                // what PostStep / Schedule report back to the runtime
  int64_t seq_id; int64_t req_id; int index;
  int new_token;                 // -1: none
  bool finished; int code; std::string message;
};

struct StepPlan {
  std::vector<int64_t> seq_ids;            // multi-token sequences first, then single-token ones
  std::vector<int> q_lens, kv_lens;
  std::vector<int> input_ids, positions, slots, cu_q;
  std::vector<int> block_table; int max_blocks = 0;
  std::vector<int64_t> sample_seq_ids;     // sequences that sample this step ...
  std::vector<int> sample_rows;            // ... and the token row whose logits they use
  std::vector<BlockCopy> pre_copies;       // tail-block copies of forks decided after the previous step: they run
                                           // first, before this step's swap-outs can touch their destinations
  std::vector<SwapCopy> swap_out, swap_in;
  std::vector<BlockCopy> copies;
  int num_multi = 0, num_single = 0, num_tokens = 0, num_multi_tokens = 0, max_q_len = 0;
  // What this step's sampling needs from the logits: the largest candidate count of any sampling row
  // (max(topk, logprobs_num)), and whether a row edits the whole logits row first (repetition penalty, n-gram
  // bans). Tensor-parallel ranks use it to exchange per-shard top-k candidates instead of whole vocabulary shards.
  int sample_k = 0;
  bool sample_full = false;
  std::vector<SeqEvent> events;            // timeouts / aborts / rejections decided while planning
  bool empty() const { return seq_ids.empty(); }
  bool has_block_ops() const { return !pre_copies.empty() || !swap_out.empty() || !swap_in.empty() || !copies.empty(); }
  void Clear() { *this = StepPlan(); }
  // Flat int32 image (header + arrays) used for the single host->device upload and for
  // broadcasting the step to the other ranks / nodes.
  std::vector<int32_t> Pack() const;
  static bool Unpack(const int32_t* data, size_t n, StepPlan* out);
  // Device images written straight into (pinned) host memory, no intermediate arrays.
  // Step image: input_ids, positions, slots [num_tokens each], cu_q [nseq + 1], kv_lens [nseq],
  // block_table [nseq * max_blocks], sample_rows. Returns the number of words (StepImageWords()).
  size_t StepImageWords() const;
  size_t WriteStepImage(int32_t* dst) const;
  // Image of a pure decode step padded to `bs` sequences and `mb` blocks per sequence (the layout a captured
  // decode graph reads): ids, positions, slots (-1 padding), kv_lens [bs each], block_table [bs * mb].
  // Returns the number of words, or 0 if the plan does not fit.
  size_t WriteDecodeImage(int32_t* dst, int bs, int mb) const;
};

struct SampledToken {
  int token;
  int64_t parent_seq = -1;       // beam search: take this sibling's history before appending
};

struct SchedulerStats {
  int64_t waiting = 0, running = 0, swapped = 0;
  int64_t free_blocks = 0, used_blocks = 0, usable_blocks = 0, free_host_blocks = 0;
  int64_t total_requests = 0, finished = 0, timeouts = 0, aborted = 0, rejected = 0;
  int64_t preempt_swap = 0, preempt_recompute = 0, swap_in = 0, steps = 0;
  int64_t step_tokens = 0, input_tokens = 0, output_tokens = 0;
  CacheStats cache;
};

class Scheduler {
 public:
  Scheduler(const SchedulerConfig& cfg, int num_device_blocks, int num_host_blocks);

  // Creates max(num_beams, num_return_sequences, 1) sequences for one request. Returns their ids.
  Status AddRequest(int64_t req_id, const std::vector<int>& prompt, const SamplingConfig& cfg,
                    std::vector<int64_t>* seq_ids);
  void Abort(int64_t req_id);
  bool Idle();

  // Plans the next step. Returns false when there is nothing to run (plan->events may still carry
  // timeouts / aborts).
  bool Schedule(StepPlan* plan);
  // Consumes the step's sampled tokens (one per plan.sample_seq_ids entry, same order).
  void PostStep(const StepPlan& plan, const std::vector<SampledToken>& sampled, std::vector<SeqEvent>* events);

  // Pipelined stepping: PostStep in two halves, so that the next step can be planned and launched while the device
  // still runs this one. Advance(plan) - right after the step is launched - moves the cached lengths forward and
  // gives every sampling sequence a placeholder token (the real one is taken from the sampler's device buffer by the
  // next step); the following Schedule() then plans those sequences' next decode row. Resolve(plan, tokens) - when
  // the step's tokens have reached the host - puts the real tokens in place, runs the finish checks and reports the
  // events PostStep would have. A sequence that turns out to be finished may already be part of the step in flight;
  // its row there is wasted and its result ignored. Only for plans whose sampling sequences are all plain (one
  // sequence per request, no beams): CanPipeline(plan) says so.
  bool CanPipeline(const StepPlan& plan);
  void Advance(const StepPlan& plan);
  void Resolve(const StepPlan& plan, const std::vector<int>& tokens, std::vector<SeqEvent>* events);

  // Runtime hooks: stop strings and structured output need the tokenizer, which lives outside.
  void FinishSequence(int64_t seq_id, int keep_tokens, int code, const std::string& message,
                      std::vector<SeqEvent>* events);
  bool ReplaceGenerated(int64_t seq_id, const std::vector<int>& generated);
  std::vector<int> GetTokens(int64_t seq_id);
  int GetPromptLen(int64_t seq_id);

  SchedulerStats GetStats();
  bool CheckInvariants(std::string* why);
  const SchedulerConfig& config() const { return cfg_; }

 private:
  using SeqPtr = std::shared_ptr<Sequence>;
  void MergeWaitingBuffer();
  void FinishLocked(const SeqPtr& s, int code, const std::string& msg, int new_token, std::vector<SeqEvent>* ev);
  void ExpireAndAbort(int64_t now, std::vector<SeqEvent>* ev);
  void PreemptLocked(const SeqPtr& victim, StepPlan* plan);
  int BlocksNeeded(const Sequence& s) const;
  bool CheckFinishLocked(const SeqPtr& s, int token, std::vector<SeqEvent>* ev);
  void EmitSequence(const SeqPtr& s, StepPlan* plan);
  int StepTokenCap(int num_decodes) const;

  CacheManager& CacheOf(const Sequence& s) { return *caches_[static_cast<size_t>(s.seq_id % static_cast<int64_t>(caches_.size()))]; }
  // Copy and swap lists are executed by the ranks, and block ids are per rank: a device block in those lists is
  // written as rank * blocks_per_rank + block, so that each rank picks out (and un-offsets) its own entries.
  int PoolBase(const Sequence& s) const { return RankOf(s) * caches_[0]->num_device_blocks(); }
  bool SwapInQualified(CacheManager& cache, const SeqPtr& s, StepPlan* plan);
  int RankOf(const Sequence& s) const { return static_cast<int>(s.seq_id % static_cast<int64_t>(caches_.size())); }

  SchedulerConfig cfg_;
  std::vector<std::unique_ptr<CacheManager>> caches_;   // one per data-parallel rank (one in all other layouts)
  std::mutex mu_;
  std::deque<SeqPtr> waiting_buffer_, waiting_;
  std::vector<SeqPtr> running_;
  std::deque<SeqPtr> swapped_;
  std::unordered_map<int64_t, SeqPtr> by_id_;
  std::unordered_map<int64_t, std::vector<SeqPtr>> groups_;
  int64_t next_seq_id_ = 1;
  bool split_fuse_on_;
  std::vector<BlockCopy> pending_copies_;   // fork copies decided in PostStep, executed by the next step
  SchedulerStats stats_;
};

}  // namespace ksana
