#include "scheduler.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include "logger.h"

namespace ksana {

namespace {
constexpr int32_t kPlanMagic = 0x4B53504C;   // "KSPL"
inline int CeilMul(int bs, float thr) { return static_cast<int>(std::ceil(static_cast<double>(bs) * thr)); }
}  // namespace

// ---------------------------------------------------------------------------------- StepPlan
std::vector<int32_t> StepPlan::Pack() const {
  // header: magic, nseq, ntok, num_multi, num_single, num_multi_tokens, max_q_len, max_blocks,
  //         nsample, nswap_out, nswap_in, ncopies, npre_copies, sample_k, sample_full, reserved
  std::vector<int32_t> out;
  const int nseq = static_cast<int>(seq_ids.size());
  out.reserve(16 + nseq * (4 + max_blocks) + num_tokens * 3 + 64);
  out.push_back(kPlanMagic);
  out.push_back(nseq);
  out.push_back(num_tokens);
  out.push_back(num_multi);
  out.push_back(num_single);
  out.push_back(num_multi_tokens);
  out.push_back(max_q_len);
  out.push_back(max_blocks);
  out.push_back(static_cast<int>(sample_rows.size()));
  out.push_back(static_cast<int>(swap_out.size()));
  out.push_back(static_cast<int>(swap_in.size()));
  out.push_back(static_cast<int>(copies.size()));
  out.push_back(static_cast<int>(pre_copies.size()));
  out.push_back(sample_k);
  out.push_back(sample_full ? 1 : 0);
  out.push_back(0);
  auto put = [&](const std::vector<int>& v) { out.insert(out.end(), v.begin(), v.end()); };
  auto put64 = [&](const std::vector<int64_t>& v) {
    for (int64_t x : v) { out.push_back(static_cast<int32_t>(x & 0xffffffff)); out.push_back(static_cast<int32_t>(x >> 32)); }
  };
  put(input_ids); put(positions); put(slots); put(cu_q); put(q_lens); put(kv_lens); put(block_table);
  put(sample_rows);
  put64(seq_ids); put64(sample_seq_ids);
  for (auto& s : swap_out) { out.push_back(s.device_block); out.push_back(s.host_block); }
  for (auto& s : swap_in) { out.push_back(s.device_block); out.push_back(s.host_block); }
  for (auto& c : copies) { out.push_back(c.src); out.push_back(c.dst); out.push_back(c.pos_delta); }
  for (auto& c : pre_copies) { out.push_back(c.src); out.push_back(c.dst); out.push_back(c.pos_delta); }
  return out;
}

bool StepPlan::Unpack(const int32_t* d, size_t n, StepPlan* p) {
  if (n < 16 || d[0] != kPlanMagic) return false;
  p->Clear();
  const int nseq = d[1];
  p->num_tokens = d[2]; p->num_multi = d[3]; p->num_single = d[4]; p->num_multi_tokens = d[5];
  p->max_q_len = d[6]; p->max_blocks = d[7];
  const int nsample = d[8], nso = d[9], nsi = d[10], ncp = d[11], npre = d[12];
  p->sample_k = d[13];
  p->sample_full = d[14] != 0;
  if (nseq < 0 || p->num_tokens < 0 || p->max_blocks < 0 || nsample < 0 || nso < 0 || nsi < 0 || ncp < 0 || npre < 0)
    return false;
  size_t need = 16 + static_cast<size_t>(p->num_tokens) * 3 + (nseq + 1) + nseq * 2 +
                static_cast<size_t>(nseq) * p->max_blocks + nsample + 2 * nseq + 2 * nsample + 2 * nso + 2 * nsi +
                3 * ncp + 3 * npre;
  if (n < need) return false;
  const int32_t* c = d + 16;
  auto get = [&](std::vector<int>* v, size_t cnt) { v->assign(c, c + cnt); c += cnt; };
  auto get64 = [&](std::vector<int64_t>* v, size_t cnt) {
    v->resize(cnt);
    for (size_t i = 0; i < cnt; ++i) {
      (*v)[i] = static_cast<int64_t>(static_cast<uint32_t>(c[0])) | (static_cast<int64_t>(c[1]) << 32);
      c += 2;
    }
  };
  get(&p->input_ids, p->num_tokens); get(&p->positions, p->num_tokens); get(&p->slots, p->num_tokens);
  get(&p->cu_q, nseq + 1); get(&p->q_lens, nseq); get(&p->kv_lens, nseq);
  get(&p->block_table, static_cast<size_t>(nseq) * p->max_blocks);
  get(&p->sample_rows, nsample);
  get64(&p->seq_ids, nseq); get64(&p->sample_seq_ids, nsample);
  for (int i = 0; i < nso; ++i) { p->swap_out.push_back({c[0], c[1]}); c += 2; }
  for (int i = 0; i < nsi; ++i) { p->swap_in.push_back({c[0], c[1]}); c += 2; }
  for (int i = 0; i < ncp; ++i) { p->copies.push_back({c[0], c[1], c[2]}); c += 3; }
  for (int i = 0; i < npre; ++i) { p->pre_copies.push_back({c[0], c[1], c[2]}); c += 3; }
  return true;
}

size_t StepPlan::StepImageWords() const {
  return static_cast<size_t>(num_tokens) * 3 + cu_q.size() + kv_lens.size() + block_table.size() + sample_rows.size();
}

size_t StepPlan::WriteStepImage(int32_t* dst) const {
  int32_t* c = dst;
  auto put = [&](const std::vector<int>& v) { if (!v.empty()) std::memcpy(c, v.data(), v.size() * sizeof(int32_t)); c += v.size(); };
  put(input_ids); put(positions); put(slots); put(cu_q); put(kv_lens); put(block_table); put(sample_rows);
  return static_cast<size_t>(c - dst);
}

size_t StepPlan::WriteDecodeImage(int32_t* dst, int bs, int mb) const {
  const int nseq = static_cast<int>(seq_ids.size());
  if (num_multi != 0 || nseq > bs || max_blocks > mb || num_tokens != nseq) return 0;
  const size_t total = static_cast<size_t>(4) * bs + static_cast<size_t>(bs) * mb;
  std::memset(dst, 0, total * sizeof(int32_t));
  std::memcpy(dst, input_ids.data(), nseq * sizeof(int32_t));
  std::memcpy(dst + bs, positions.data(), nseq * sizeof(int32_t));
  for (int i = 0; i < bs; ++i) dst[2 * bs + i] = i < nseq ? slots[i] : -1;
  std::memcpy(dst + 3 * bs, kv_lens.data(), nseq * sizeof(int32_t));
  int32_t* tbl = dst + 4 * bs;
  for (int i = 0; i < nseq; ++i)
    std::memcpy(tbl + static_cast<size_t>(i) * mb, block_table.data() + static_cast<size_t>(i) * max_blocks,
                max_blocks * sizeof(int32_t));
  return total;
}

// --------------------------------------------------------------------------------- Scheduler
Scheduler::Scheduler(const SchedulerConfig& cfg, int num_device_blocks, int num_host_blocks)
    : cfg_(cfg), split_fuse_on_(cfg.split_fuse_token_num > 0) {
  for (int r = 0; r < std::max(1, cfg.dp_size); ++r)
    caches_.emplace_back(new CacheManager(num_device_blocks, num_host_blocks, cfg.block_token_num, cfg.enable_prefix_cache));
  if (cfg_.max_step_tokens < cfg_.max_batch_size) cfg_.max_step_tokens = cfg_.max_batch_size;
}

Status Scheduler::AddRequest(int64_t req_id, const std::vector<int>& prompt, const SamplingConfig& in_cfg,
                             std::vector<int64_t>* seq_ids) {
  auto cfg = std::make_shared<SamplingConfig>(in_cfg);
  Status st = cfg->VerifyArgs();
  if (!st.ok()) return st;
  if (prompt.empty()) return Status(RET_INVALID_ARGUMENT, "empty input tokens");
  if (static_cast<int>(prompt.size()) > cfg_.max_token_len) {
    std::lock_guard<std::mutex> g(mu_);
    ++stats_.rejected;
    return Status(RET_EXCEED_LENGTH, "input length " + std::to_string(prompt.size()) + " exceeds max_token_len " +
                                         std::to_string(cfg_.max_token_len));
  }
  const int n = std::max({cfg->num_beams, cfg->num_return_sequences, 1});
  std::lock_guard<std::mutex> g(mu_);
  if (static_cast<int>(waiting_buffer_.size() + waiting_.size()) >= cfg_.max_waiting_queue_len) {
    ++stats_.rejected;
    KLLM_LOG_WARNING << "req " << req_id << " rejected: waiting queue is full (" << cfg_.max_waiting_queue_len << ")";
    return Status(RET_EXCEED_CAPACITY, "waiting queue is full");
  }
  ++stats_.total_requests;
  stats_.input_tokens += static_cast<int64_t>(prompt.size());
  const int64_t now = NowMs();
  std::vector<SeqPtr> group;
  for (int i = 0; i < n; ++i) {
    auto s = std::make_shared<Sequence>();
    // siblings share blocks with the leader, so they live on its rank: ids one rank-stride apart
    s->seq_id = i == 0 ? next_seq_id_ : group[0]->seq_id + static_cast<int64_t>(i) * static_cast<int64_t>(caches_.size());
    next_seq_id_ = std::max(next_seq_id_, s->seq_id + 1);
    s->req_id = req_id;
    s->index = i;
    s->tokens = prompt;
    s->prompt_len = static_cast<int>(prompt.size());
    s->cfg = cfg;
    s->arrive_ms = now;
    if (i > 0) { s->forked_pending = true; s->leader = group[0]->seq_id; }
    group.push_back(s);
    seq_ids->push_back(s->seq_id);
  }
  for (auto& s : group) by_id_[s->seq_id] = s;
  groups_[req_id] = group;
  waiting_buffer_.push_back(group[0]);   // siblings join when the leader's prefill completes
  return Status();
}

void Scheduler::Abort(int64_t req_id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = groups_.find(req_id);
  if (it == groups_.end()) return;
  for (auto& s : it->second) s->aborted = true;
}

bool Scheduler::Idle() {
  std::lock_guard<std::mutex> g2(mu_);
  return waiting_buffer_.empty() && waiting_.empty() && running_.empty() && swapped_.empty();
}

void Scheduler::MergeWaitingBuffer() {
  while (!waiting_buffer_.empty()) {
    waiting_.push_back(waiting_buffer_.front());
    waiting_buffer_.pop_front();
  }
}

void Scheduler::FinishLocked(const SeqPtr& s, int code, const std::string& msg, int new_token,
                             std::vector<SeqEvent>* ev) {
  if (s->state == SeqState::FINISHED) return;
  CacheOf(*s).Release(s->blocks);
  s->blocks.clear();
  CacheOf(*s).ReleaseHost(s->host_blocks);
  s->host_blocks.clear();
  s->state = SeqState::FINISHED;
  s->finish_status = Status(static_cast<RetCode>(code), msg);
  ++stats_.finished;
  if (ev) ev->push_back({s->seq_id, s->req_id, s->index, new_token, true, code, msg});
  by_id_.erase(s->seq_id);
  auto git = groups_.find(s->req_id);
  if (git != groups_.end()) {
    bool all = true;
    for (auto& m : git->second) all = all && m->state == SeqState::FINISHED;
    if (all) groups_.erase(git);
  }
}

void Scheduler::ExpireAndAbort(int64_t now, std::vector<SeqEvent>* ev) {
  auto dead = [&](const SeqPtr& s, bool queued) -> bool {
    if (s->aborted) {
      ++stats_.aborted;
      // pending siblings of an aborted leader never ran: finish them too
      auto git = groups_.find(s->req_id);
      std::vector<SeqPtr> sibs;
      if (git != groups_.end()) sibs = git->second;
      FinishLocked(s, RET_TERMINATED, "client aborted.", -1, ev);
      for (auto& m : sibs)
        if (m->forked_pending && m->state != SeqState::FINISHED) FinishLocked(m, RET_TERMINATED, "client aborted.", -1, ev);
      return true;
    }
    if (queued && now >= s->arrive_ms + cfg_.waiting_timeout_in_ms) {
      ++stats_.timeouts;
      KLLM_LOG_WARNING << "req " << s->req_id << " waited " << (now - s->arrive_ms) << " ms in the queue: timeout";
      auto git = groups_.find(s->req_id);
      std::vector<SeqPtr> sibs;
      if (git != groups_.end()) sibs = git->second;
      FinishLocked(s, RET_TIMEOUT, "running timeout.", -1, ev);
      for (auto& m : sibs)
        if (m->forked_pending && m->state != SeqState::FINISHED) FinishLocked(m, RET_TIMEOUT, "running timeout.", -1, ev);
      return true;
    }
    return false;
  };
  running_.erase(std::remove_if(running_.begin(), running_.end(), [&](const SeqPtr& s) { return dead(s, false); }),
                 running_.end());
  swapped_.erase(std::remove_if(swapped_.begin(), swapped_.end(), [&](const SeqPtr& s) { return dead(s, true); }),
                 swapped_.end());
  waiting_.erase(std::remove_if(waiting_.begin(), waiting_.end(), [&](const SeqPtr& s) { return dead(s, true); }),
                 waiting_.end());
}

int Scheduler::BlocksNeeded(const Sequence& s) const {
  const int target = CeilDiv(s.kv_cached + s.chunk, cfg_.block_token_num);
  return std::max(0, target - static_cast<int>(s.blocks.size()));
}

int Scheduler::StepTokenCap(int num_decodes) const {
  int cap = cfg_.max_step_tokens;
  if (split_fuse_on_) cap = std::min(cap, std::max(cfg_.split_fuse_token_num, num_decodes + cfg_.block_token_num));
  return cap;
}

void Scheduler::PreemptLocked(const SeqPtr& v, StepPlan* plan) {
  ++v->preempt_count;
  KLLM_LOG_DEBUG << "preempt seq " << v->seq_id << " (req " << v->req_id << ", " << v->blocks.size() << " blocks, mode "
                 << (cfg_.preempt_mode == 0 ? "swap" : "recompute") << ")";
  const size_t so0 = plan->swap_out.size();
  if (cfg_.preempt_mode == 0 && CacheOf(*v).SwapOut(&v->blocks, &v->host_blocks, &plan->swap_out)) {
    for (size_t i = so0; i < plan->swap_out.size(); ++i) plan->swap_out[i].device_block += PoolBase(*v);
    v->promoted = std::min(v->promoted, static_cast<int>(v->blocks.size()));
    v->state = SeqState::SWAPPED;
    swapped_.push_back(v);
    ++stats_.preempt_swap;
    return;
  }
  // recompute: everything generated so far becomes the prompt of a fresh prefill
  CacheOf(*v).Release(v->blocks);
  v->blocks.clear();
  v->kv_cached = 0;
  v->promoted = 0;
  v->chunk = 0;
  v->state = SeqState::WAITING;
  waiting_.push_front(v);
  ++stats_.preempt_recompute;
}

void Scheduler::EmitSequence(const SeqPtr& s, StepPlan* plan) {
  const int B = cfg_.block_token_num;
  plan->seq_ids.push_back(s->seq_id);
  plan->q_lens.push_back(s->chunk);
  plan->kv_lens.push_back(s->kv_cached + s->chunk);
  for (int i = 0; i < s->chunk; ++i) {
    const int pos = s->kv_cached + i;
    plan->input_ids.push_back(s->tokens[pos]);
    plan->positions.push_back(pos);
    plan->slots.push_back(s->blocks[pos / B] * B + pos % B);
  }
  plan->num_tokens += s->chunk;
  plan->max_q_len = std::max(plan->max_q_len, s->chunk);
  if (s->kv_cached + s->chunk == static_cast<int>(s->tokens.size())) {
    const int row = plan->num_tokens - 1;
    plan->sample_seq_ids.push_back(s->seq_id);
    plan->sample_rows.push_back(row);
    const SamplingConfig& c = *s->cfg;
    plan->sample_k = std::max(plan->sample_k, std::max(c.topk, c.logprobs_num));
    if (c.repetition_penalty != 1.0f || c.no_repeat_ngram_size > 0 || c.encoder_no_repeat_ngram_size > 0)
      plan->sample_full = true;
    // siblings waiting for this prefill draw their first token from the same logits row
    auto git = groups_.find(s->req_id);
    if (git != groups_.end()) {
      for (auto& m : git->second) {
        if (m->forked_pending && m->leader == s->seq_id && m->state != SeqState::FINISHED) {
          plan->sample_seq_ids.push_back(m->seq_id);
          plan->sample_rows.push_back(row);
        }
      }
    }
  }
}

bool Scheduler::SwapInQualified(CacheManager& cache, const SeqPtr& s, StepPlan* plan) {
  const size_t n0 = plan->swap_in.size();
  if (!cache.SwapIn(&s->blocks, &s->host_blocks, &plan->swap_in)) return false;
  for (size_t i = n0; i < plan->swap_in.size(); ++i) plan->swap_in[i].device_block += PoolBase(*s);
  return true;
}

bool Scheduler::Schedule(StepPlan* plan) {
  std::lock_guard<std::mutex> g(mu_);
  MergeWaitingBuffer();
  plan->Clear();
  const int64_t now = NowMs();
  const int B = cfg_.block_token_num;
  ExpireAndAbort(now, &plan->events);

  // ------------------------------------------------------------------ running queue
  int num_decodes = 0;
  for (auto& s : running_) num_decodes += (!s->draining && static_cast<int>(s->tokens.size()) - s->kv_cached == 1);
  int cap = StepTokenCap(num_decodes);
  int step_tokens = 0;
  for (auto& s : running_) {
    if (s->draining) { s->chunk = 0; continue; }     // its last token is still on the device: nothing more to run
    const int remaining = static_cast<int>(s->tokens.size()) - s->kv_cached;
    int chunk = std::min(remaining, std::max(cap - step_tokens, 0));
    if (chunk < remaining) chunk = ((s->kv_cached + chunk) / B) * B - s->kv_cached;   // chunks end on block boundaries
    s->chunk = std::max(chunk, 0);
    step_tokens += s->chunk;
  }
  // a sequence that got no token budget this step (chunk == 0) simply idles until the next one
  // per data-parallel rank: blocks this step needs and sequences running there (one rank in all other layouts)
  const int R = static_cast<int>(caches_.size());
  std::vector<int> rank_need(R, 0), rank_bs(R, 0);
  for (auto& s : running_) { rank_need[RankOf(*s)] += BlocksNeeded(*s); ++rank_bs[RankOf(*s)]; }
  bool step_sched_finish = false;
  for (int r = 0; r < R; ++r) {
    while (rank_bs[r] > 0) {
      const int usable = caches_[r]->usable_blocks();
      if (rank_need[r] + CeilMul(rank_bs[r], cfg_.swapout_block_threshold) <= usable) break;
      // the youngest sequence of this rank goes first
      int vi = static_cast<int>(running_.size()) - 1;
      while (vi >= 0 && RankOf(*running_[vi]) != r) --vi;
      if (vi < 0) break;
      SeqPtr v = running_[vi];
      if (rank_bs[r] == 1) {
        if (rank_need[r] <= usable) break;
        // a lone request that cannot grow any more can never finish
        running_.erase(running_.begin() + vi);
        KLLM_LOG_WARNING << "req " << v->req_id << ": not enough KV cache blocks for a single sequence of "
                         << v->tokens.size() << " tokens; finishing it with RET_OUT_OF_MEMORY";
        FinishLocked(v, RET_OUT_OF_MEMORY, "not enough KV cache blocks for this request", -1, &plan->events);
        rank_need[r] = 0;
        rank_bs[r] = 0;
        break;
      }
      running_.erase(running_.begin() + vi);
      rank_need[r] -= BlocksNeeded(*v);
      --rank_bs[r];
      step_tokens -= v->chunk;
      if (split_fuse_on_ && cfg_.split_fuse_token_num > 0) split_fuse_on_ = false;   // memory pressure: stop chunk-mixing
      PreemptLocked(v, plan);
      step_sched_finish = true;
    }
  }
  for (auto& s : running_) {
    const bool ok = CacheOf(*s).Allocate(BlocksNeeded(*s), &s->blocks);
    if (!ok) { s->chunk = 0; }   // cannot happen after the check above; keep the step consistent anyway
  }

  // ------------------------------------------------------------------ swapped queue
  if (!step_sched_finish && cfg_.preempt_mode == 0) {
    while (!swapped_.empty()) {
      SeqPtr s = swapped_.front();
      const int bs = static_cast<int>(running_.size());
      int bs_rank = 0;                                   // block thresholds count the sequences of the same rank
      for (auto& o : running_) bs_rank += (RankOf(*o) == RankOf(*s));
      CacheManager& cache = CacheOf(*s);
      const int remaining = static_cast<int>(s->tokens.size()) - s->kv_cached;
      s->chunk = remaining;
      const int need = static_cast<int>(s->host_blocks.size()) +
                       std::max(0, CeilDiv(s->kv_cached + s->chunk, B) -
                                       static_cast<int>(s->blocks.size() + s->host_blocks.size()));
      if (bs + 1 <= cfg_.max_batch_size && step_tokens + s->chunk <= cap &&
          need + CeilMul(bs_rank, cfg_.swapin_block_threshold) <= cache.usable_blocks() &&
          SwapInQualified(cache, s, plan)) {
        cache.Allocate(BlocksNeeded(*s), &s->blocks);
        s->promoted = cache.Promote(s->tokens, &s->blocks, s->kv_cached, s->promoted);
        s->state = SeqState::RUNNING;
        running_.push_back(s);
        swapped_.pop_front();
        step_tokens += s->chunk;
        ++stats_.swap_in;
      } else {
        step_sched_finish = true;   // swapped requests have priority over new ones
        break;
      }
    }
  }

  // ------------------------------------------------------------------ waiting queue
  const bool static_batching = cfg_.schedule_strategy == 1;
  bool admit = !step_sched_finish;
  if (static_batching && admit) {
    // static batching: gather for a while, then run the gathered batch to completion
    if (!running_.empty()) admit = false;
    else if (!waiting_.empty() && static_cast<int>(waiting_.size()) < cfg_.max_batch_size &&
             now - waiting_.front()->arrive_ms < cfg_.auto_batch_wait_ms) admit = false;
  }
  while (admit && !waiting_.empty()) {
    SeqPtr s = waiting_.front();
    const int len = static_cast<int>(s->tokens.size());
    int siblings = 0;
    auto git = groups_.find(s->req_id);
    if (git != groups_.end())
      for (auto& m : git->second) siblings += (m->forked_pending && m->leader == s->seq_id);
    const int bs = static_cast<int>(running_.size());
    if (bs + 1 + siblings > cfg_.max_batch_size) break;
    int bs_rank = 0;
    for (auto& o : running_) bs_rank += (RankOf(*o) == RankOf(*s));
    CacheManager& cache = CacheOf(*s);
    // cached prefix (re-evaluated at every attempt: the tree may have changed meanwhile)
    std::vector<int> pre_blocks;
    std::vector<BlockCopy> flex_copies;
    int matched = cache.AcquirePrefix(s->tokens, &pre_blocks);
    int flex = 0;
    if (cfg_.min_flexible_cache_num > 0)
      flex = cache.AcquireFlexible(s->tokens, matched, cfg_.min_flexible_cache_num, &pre_blocks, &flex_copies);
    const int cached = std::min(matched + flex, len - 1);    // at least the last token is computed
    const int remaining = len - cached;
    int chunk = std::min(remaining, std::max(cap - step_tokens, 0));
    if (chunk < remaining) chunk = ((cached + chunk) / B) * B - cached;
    const int unique = std::max(0, CeilDiv(cached + std::max(chunk, 0), B) - static_cast<int>(pre_blocks.size()));
    if (chunk <= 0 || unique + CeilMul(bs_rank, cfg_.launch_block_threshold) > cache.usable_blocks()) {
      cache.Release(pre_blocks);
      break;   // FIFO: nobody overtakes the head
    }
    s->blocks = pre_blocks;
    s->kv_cached = cached;
    s->prefix_hit_tokens = matched;
    s->flexible_hit_tokens = flex;
    s->promoted = matched / B;
    s->chunk = chunk;
    cache.Allocate(unique, &s->blocks);
    for (auto& c : flex_copies) plan->copies.push_back({c.src + PoolBase(*s), c.dst + PoolBase(*s), c.pos_delta});
    s->state = SeqState::RUNNING;
    running_.push_back(s);
    waiting_.pop_front();
    step_tokens += chunk;
  }

  // ------------------------------------------------------------------ emit (multi-token first)
  std::vector<SeqPtr> multi, single;
  for (auto& s : running_) {
    if (s->chunk <= 0) continue;
    (s->chunk > 1 ? multi : single).push_back(s);
  }
  plan->cu_q.push_back(0);
  for (auto& s : multi) { EmitSequence(s, plan); plan->cu_q.push_back(plan->num_tokens); }
  plan->num_multi = static_cast<int>(multi.size());
  plan->num_multi_tokens = plan->num_tokens;
  for (auto& s : single) { EmitSequence(s, plan); plan->cu_q.push_back(plan->num_tokens); }
  plan->num_single = static_cast<int>(single.size());
  int max_blocks = 1;
  for (auto& s : multi) max_blocks = std::max(max_blocks, static_cast<int>(s->blocks.size()));
  for (auto& s : single) max_blocks = std::max(max_blocks, static_cast<int>(s->blocks.size()));
  plan->max_blocks = max_blocks;
  plan->block_table.assign(static_cast<size_t>(plan->seq_ids.size()) * max_blocks, 0);
  size_t row = 0;
  auto fill = [&](const SeqPtr& s) {
    std::copy(s->blocks.begin(), s->blocks.end(), plan->block_table.begin() + row * max_blocks);
    ++row;
  };
  for (auto& s : multi) fill(s);
  for (auto& s : single) fill(s);

  if (!pending_copies_.empty()) {
    // Forks decided after the previous step: their tail-block copies run first, before this step's swap-outs,
    // swap-ins and copies. A fork's destination block may be swapped out (its owner is the youngest sequence, the
    // first victim) or freed and handed out again by this very plan, so it has to be filled before any of that.
    plan->pre_copies.swap(pending_copies_);
    pending_copies_.clear();
  }
  ++stats_.steps;
  stats_.step_tokens += plan->num_tokens;
  return !plan->empty() || plan->has_block_ops();
}

bool Scheduler::CheckFinishLocked(const SeqPtr& s, int token, std::vector<SeqEvent>* ev) {
  const SamplingConfig& c = *s->cfg;
  const int generated = static_cast<int>(s->tokens.size()) - s->prompt_len;
  bool stop = std::find(c.stop_token_ids.begin(), c.stop_token_ids.end(), token) != c.stop_token_ids.end();
  if (!stop && !c.ignore_eos)
    stop = std::find(cfg_.eos_token_ids.begin(), cfg_.eos_token_ids.end(), token) != cfg_.eos_token_ids.end();
  if (stop || generated >= c.max_new_tokens || static_cast<int>(s->tokens.size()) >= cfg_.max_token_len) {
    FinishLocked(s, RET_SUCCESS, "", token, ev);
    return true;
  }
  return false;
}

void Scheduler::PostStep(const StepPlan& plan, const std::vector<SampledToken>& sampled, std::vector<SeqEvent>* ev) {
  std::lock_guard<std::mutex> g(mu_);
  const int64_t now = NowMs();
  // 1. every forwarded sequence advances its cached length and publishes its full blocks
  for (size_t i = 0; i < plan.seq_ids.size(); ++i) {
    auto it = by_id_.find(plan.seq_ids[i]);
    if (it == by_id_.end()) continue;
    SeqPtr s = it->second;
    if (s->state != SeqState::RUNNING) continue;
    s->kv_cached += plan.q_lens[i];
    s->chunk = 0;
    s->promoted = CacheOf(*s).Promote(s->tokens, &s->blocks, s->kv_cached, s->promoted);
  }
  // 2. beam re-parenting uses the parents' state before any token of this step is appended
  struct Reparent { SeqPtr dst; std::vector<int> tokens; std::vector<int> blocks; int kv; int promoted; };
  std::vector<Reparent> moves;
  std::vector<BlockCopy> fork_copies;
  for (size_t i = 0; i < plan.sample_seq_ids.size() && i < sampled.size(); ++i) {
    const int64_t pid = sampled[i].parent_seq;
    if (pid < 0 || pid == plan.sample_seq_ids[i]) continue;
    auto dit = by_id_.find(plan.sample_seq_ids[i]);
    auto pit = by_id_.find(pid);
    if (dit == by_id_.end() || pit == by_id_.end()) continue;
    Reparent mv{dit->second, pit->second->tokens, {}, pit->second->kv_cached, 0};
    if (RankOf(*dit->second) != RankOf(*pit->second)) continue;          // beams of a group share a rank by construction
    const size_t fc0 = fork_copies.size();
    if (!CacheOf(*pit->second).Fork(pit->second->blocks, pit->second->kv_cached, &mv.blocks, &fork_copies)) continue;
    for (size_t k = fc0; k < fork_copies.size(); ++k) { fork_copies[k].src += PoolBase(*pit->second); fork_copies[k].dst += PoolBase(*pit->second); }
    mv.promoted = std::min(pit->second->promoted, pit->second->kv_cached / cfg_.block_token_num);
    moves.push_back(std::move(mv));
  }
  for (auto& mv : moves) {
    CacheOf(*mv.dst).Release(mv.dst->blocks);
    mv.dst->blocks = std::move(mv.blocks);
    mv.dst->tokens = std::move(mv.tokens);
    mv.dst->kv_cached = mv.kv;
    mv.dst->promoted = mv.promoted;
  }
  pending_copies_.insert(pending_copies_.end(), fork_copies.begin(), fork_copies.end());
  // 3. append sampled tokens, start pending siblings, finish what is done
  for (size_t i = 0; i < plan.sample_seq_ids.size() && i < sampled.size(); ++i) {
    auto it = by_id_.find(plan.sample_seq_ids[i]);
    if (it == by_id_.end()) continue;
    SeqPtr s = it->second;
    if (s->state == SeqState::FINISHED) continue;
    if (s->forked_pending) {
      auto lit = by_id_.find(s->leader);
      // the leader may already have finished in this very loop (e.g. max_new_tokens == 1): its
      // blocks were released but are still intact, yet no longer safe to share -> recompute path
      if (lit != by_id_.end() && lit->second->state == SeqState::RUNNING) {
        SeqPtr l = lit->second;
        // leader appended its own token already when it precedes us; share only the prompt part
        const int shared_tokens = std::min(l->kv_cached, s->prompt_len);
        std::vector<BlockCopy> cps;
        if (RankOf(*l) == RankOf(*s) && CacheOf(*l).Fork(l->blocks, shared_tokens, &s->blocks, &cps)) {
          for (auto& c : cps) { c.src += PoolBase(*l); c.dst += PoolBase(*l); }
          pending_copies_.insert(pending_copies_.end(), cps.begin(), cps.end());
          s->kv_cached = shared_tokens;
          s->promoted = std::min(l->promoted, shared_tokens / cfg_.block_token_num);
        }
      }
      s->forked_pending = false;
      s->state = SeqState::RUNNING;
      running_.push_back(s);
    }
    if (s->sampled == 0) s->first_token_ms = now;
    ++s->sampled;
    s->tokens.push_back(sampled[i].token);
    ++stats_.output_tokens;
    if (!CheckFinishLocked(s, sampled[i].token, ev)) {
      ev->push_back({s->seq_id, s->req_id, s->index, sampled[i].token, false, 0, ""});
    }
  }
  running_.erase(std::remove_if(running_.begin(), running_.end(),
                                [](const SeqPtr& s) { return s->state == SeqState::FINISHED; }),
                 running_.end());
}

bool Scheduler::CanPipeline(const StepPlan& plan) {
  std::lock_guard<std::mutex> g(mu_);
  for (int64_t id : plan.sample_seq_ids) {
    auto it = by_id_.find(id);
    if (it == by_id_.end()) continue;
    const Sequence& s = *it->second;
    if (s.forked_pending || s.cfg->num_beams > 1) return false;
    auto git = groups_.find(s.req_id);
    if (git != groups_.end() && git->second.size() > 1) return false;      // siblings fork on sampled results
  }
  return true;
}

void Scheduler::Advance(const StepPlan& plan) {
  std::lock_guard<std::mutex> g(mu_);
  for (size_t i = 0; i < plan.seq_ids.size(); ++i) {
    auto it = by_id_.find(plan.seq_ids[i]);
    if (it == by_id_.end()) continue;
    SeqPtr s = it->second;
    if (s->state != SeqState::RUNNING) continue;
    s->kv_cached += plan.q_lens[i];
    s->chunk = 0;
    // every token up to kv_cached is a real one here (the previous step was resolved before this call)
    s->promoted = CacheOf(*s).Promote(s->tokens, &s->blocks, s->kv_cached, s->promoted);
  }
  for (int64_t id : plan.sample_seq_ids) {
    auto it = by_id_.find(id);
    if (it == by_id_.end()) continue;
    SeqPtr s = it->second;
    if (s->state == SeqState::FINISHED || s->token_pending) continue;
    s->tokens.push_back(-1);
    s->token_pending = true;
    const int generated = static_cast<int>(s->tokens.size()) - s->prompt_len;
    s->draining = generated >= s->cfg->max_new_tokens || static_cast<int>(s->tokens.size()) >= cfg_.max_token_len;
  }
}

void Scheduler::Resolve(const StepPlan& plan, const std::vector<int>& tokens, std::vector<SeqEvent>* ev) {
  std::lock_guard<std::mutex> g(mu_);
  const int64_t now = NowMs();
  for (size_t i = 0; i < plan.sample_seq_ids.size() && i < tokens.size(); ++i) {
    auto it = by_id_.find(plan.sample_seq_ids[i]);
    if (it == by_id_.end()) continue;                 // finished or aborted meanwhile: the row was wasted work
    SeqPtr s = it->second;
    if (s->state == SeqState::FINISHED || !s->token_pending || s->tokens.empty()) continue;
    s->tokens.back() = tokens[i];
    s->token_pending = false;
    s->draining = false;
    if (s->sampled == 0) s->first_token_ms = now;
    ++s->sampled;
    ++stats_.output_tokens;
    if (!CheckFinishLocked(s, tokens[i], ev)) ev->push_back({s->seq_id, s->req_id, s->index, tokens[i], false, 0, ""});
  }
  running_.erase(std::remove_if(running_.begin(), running_.end(),
                                [](const SeqPtr& s) { return s->state == SeqState::FINISHED; }),
                 running_.end());
}

void Scheduler::FinishSequence(int64_t seq_id, int keep_tokens, int code, const std::string& message,
                               std::vector<SeqEvent>* ev) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_id_.find(seq_id);
  if (it == by_id_.end()) return;
  SeqPtr s = it->second;
  if (keep_tokens >= 0 && keep_tokens < static_cast<int>(s->tokens.size())) s->tokens.resize(keep_tokens);
  FinishLocked(s, code, message, -1, ev);
  running_.erase(std::remove(running_.begin(), running_.end(), s), running_.end());
  swapped_.erase(std::remove(swapped_.begin(), swapped_.end(), s), swapped_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), s), waiting_.end());
}

bool Scheduler::ReplaceGenerated(int64_t seq_id, const std::vector<int>& generated) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_id_.find(seq_id);
  if (it == by_id_.end()) return false;
  SeqPtr s = it->second;
  // keep the longest common prefix of the old and new generated text cached
  const int old_len = static_cast<int>(s->tokens.size());
  int common = s->prompt_len;
  while (common < old_len && common - s->prompt_len < static_cast<int>(generated.size()) &&
         s->tokens[common] == generated[common - s->prompt_len]) ++common;
  s->tokens.resize(s->prompt_len);
  s->tokens.insert(s->tokens.end(), generated.begin(), generated.end());
  const int B = cfg_.block_token_num;
  const int new_cached = std::min({s->kv_cached, common, static_cast<int>(s->tokens.size()) - 1});
  if (new_cached < s->kv_cached) {
    // blocks past the divergence point may be shared through the tree: give them back and let the
    // next step allocate private ones
    const int keep_blocks = new_cached / B;   // whole blocks that stay valid
    if (keep_blocks < static_cast<int>(s->blocks.size())) {
      std::vector<int> drop(s->blocks.begin() + keep_blocks, s->blocks.end());
      CacheOf(*s).Release(drop);
      s->blocks.resize(keep_blocks);
    }
    s->kv_cached = keep_blocks * B;
    s->promoted = std::min(s->promoted, keep_blocks);
  }
  return true;
}

std::vector<int> Scheduler::GetTokens(int64_t seq_id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_id_.find(seq_id);
  return it == by_id_.end() ? std::vector<int>() : it->second->tokens;
}

int Scheduler::GetPromptLen(int64_t seq_id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_id_.find(seq_id);
  return it == by_id_.end() ? -1 : it->second->prompt_len;
}

SchedulerStats Scheduler::GetStats() {
  std::lock_guard<std::mutex> g2(mu_);
  SchedulerStats s = stats_;
  s.waiting = static_cast<int64_t>(waiting_.size() + waiting_buffer_.size());
  s.running = static_cast<int64_t>(running_.size());
  s.swapped = static_cast<int64_t>(swapped_.size());
  // the tightest rank for the pools, the sum for the counters
  s.free_blocks = caches_[0]->free_blocks();
  s.usable_blocks = caches_[0]->usable_blocks();
  s.used_blocks = caches_[0]->used_blocks();
  s.free_host_blocks = caches_[0]->free_host_blocks();
  s.cache = caches_[0]->stats();
  for (size_t r = 1; r < caches_.size(); ++r) {
    s.free_blocks = std::min<int64_t>(s.free_blocks, caches_[r]->free_blocks());
    s.usable_blocks = std::min<int64_t>(s.usable_blocks, caches_[r]->usable_blocks());
    s.used_blocks = std::max<int64_t>(s.used_blocks, caches_[r]->used_blocks());
    s.free_host_blocks = std::min<int64_t>(s.free_host_blocks, caches_[r]->free_host_blocks());
    s.cache += caches_[r]->stats();
  }
  return s;
}

bool Scheduler::CheckInvariants(std::string* why) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& c : caches_)
    if (!c->CheckInvariants(why)) return false;
  return true;
}

}  // namespace ksana
