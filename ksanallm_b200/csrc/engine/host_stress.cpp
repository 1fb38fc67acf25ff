// Stand-alone stress driver of the host runtime for sanitizer builds (ThreadSanitizer / AddressSanitizer):
//   python -m ksanallm_b200.build --sanitizer thread     ->  ksanallm_b200/build/host_stress_thread
// 1. Scheduler + cache manager under concurrency: client threads add and abort requests while one engine thread
//    plans steps and feeds back fake tokens; a small block pool forces preemption, swap-out / swap-in and prefix
//    sharing. At the end every request is finished and the block accounting invariants hold.
// 2. Control plane: a master and two workers over localhost TCP (registration, barrier, layer assignment,
//    block-number consensus, step-plan broadcast, heartbeats, cluster shutdown), each on its own thread.
// 3. Loop thread: several producers hand work to a BatchLoop and wake it while it sleeps, a failing step goes through
//    the error callable, Stop() joins. 4. OTLP exporter: spans and metric snapshots enqueued from several threads for a
//    collector that is not there (connection refused): everything is dropped and counted, nothing blocks.
// The reference ships no sanitizer configuration (only gcov flags: CMakeLists.txt WITH_TESTING); its scheduler is
// guarded by two hand-placed mutexes (src/ksana_llm/batch_scheduler/state/batch_state.h).
#include <atomic>
#include <cstdio>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "batch_loop.h"
#include "control_channel.h"
#include "otlp_export.h"
#include "scheduler.h"
#include "waiter.h"

using namespace ksana;

static int g_failures = 0;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) { std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_failures; } \
  } while (0)

static void SchedulerStress(int preempt_mode, int dp_size = 1) {
  SchedulerConfig cfg;
  cfg.dp_size = dp_size;                  // > 1: one block pool per data-parallel rank
  cfg.max_batch_size = 16;
  cfg.max_step_tokens = 256;
  cfg.max_token_len = 224;
  cfg.launch_block_threshold = 0.25f;     // admit eagerly so that growing sequences run out of blocks
  cfg.max_waiting_queue_len = 4096;
  cfg.enable_prefix_cache = true;
  cfg.split_fuse_token_num = 64;
  cfg.preempt_mode = preempt_mode;
  cfg.block_token_num = 16;
  cfg.eos_token_ids = {2};
  Scheduler sched(cfg, /*device blocks*/ 40, /*host blocks*/ preempt_mode == 0 ? 64 : 0);
  constexpr int kClients = 4, kPerClient = 40;
  std::atomic<int> added{0}, finished{0}, rejected{0};
  std::atomic<bool> clients_done{false};
  std::vector<std::thread> clients;
  for (int c = 0; c < kClients; ++c) {
    clients.emplace_back([&, c] {
      std::mt19937 rng(1234 + c);
      for (int i = 0; i < kPerClient; ++i) {
        const int64_t req_id = c * 1000 + i + 1;
        std::vector<int> prompt(8 + rng() % 90);
        for (size_t k = 0; k < prompt.size(); ++k) prompt[k] = 3 + (k < 32 ? static_cast<int>(k) : static_cast<int>(rng() % 200));
        SamplingConfig sc;
        sc.max_new_tokens = 16 + static_cast<int>(rng() % 100);
        sc.ignore_eos = (rng() % 2) == 0;
        if (rng() % 8 == 0) sc.num_return_sequences = 2, sc.topk = 4;
        std::vector<int64_t> ids;
        Status st = sched.AddRequest(req_id, prompt, sc, &ids);
        if (st.ok()) {
          added += static_cast<int>(ids.size());
          if (rng() % 10 == 0) sched.Abort(req_id);
        } else {
          ++rejected;
        }
        if (i % 8 == 0) std::this_thread::sleep_for(std::chrono::microseconds(200));
      }
    });
  }
  std::thread engine([&] {
    std::mt19937 rng(99);
    int idle_rounds = 0;
    while (idle_rounds < 2000) {
      StepPlan plan;
      const bool run = sched.Schedule(&plan);
      for (const SeqEvent& e : plan.events) finished += e.finished ? 1 : 0;
      if (!run) {
        if (clients_done.load() && sched.Idle()) break;
        ++idle_rounds;
        std::this_thread::sleep_for(std::chrono::microseconds(100));
        continue;
      }
      idle_rounds = 0;
      std::vector<SampledToken> sampled(plan.sample_seq_ids.size());
      for (auto& t : sampled) t.token = (rng() % 200 == 0) ? 2 : 3 + static_cast<int>(rng() % 200);
      std::vector<SeqEvent> events;
      sched.PostStep(plan, sampled, &events);
      for (const SeqEvent& e : events) finished += e.finished ? 1 : 0;
    }
  });
  for (auto& t : clients) t.join();
  clients_done = true;
  engine.join();
  std::string why;
  EXPECT(sched.CheckInvariants(&why));
  if (!why.empty()) std::fprintf(stderr, "invariants: %s\n", why.c_str());
  EXPECT(sched.Idle());
  EXPECT(finished.load() == added.load());
  const SchedulerStats st = sched.GetStats();
  std::printf("scheduler stress (preempt mode %d): %d sequences, %d rejected, %lld steps, %lld swap preemptions, %lld recompute "
              "preemptions, %lld prefix hit tokens\n", preempt_mode, added.load(), rejected.load(),
              static_cast<long long>(st.steps), static_cast<long long>(st.preempt_swap),
              static_cast<long long>(st.preempt_recompute), static_cast<long long>(st.cache.prefix_hit_tokens));
}

static void ControlPlaneStress() {
  ControlMaster master("127.0.0.1", 0, 3, /*heartbeat interval ms*/ 50, /*timeout ms*/ 2000);
  const int port = master.port();
  std::atomic<int> got{0};
  std::vector<std::thread> workers;
  for (int r = 1; r <= 2; ++r) {
    workers.emplace_back([&, r] {
      ControlWorker w("127.0.0.1", port, r, 50, 2000);
      EXPECT(w.Connect(5000));
      EXPECT(w.Barrier(5000));
      auto range = w.GetLayers(5000);
      EXPECT(range.first >= 0 && range.second >= range.first);
      EXPECT(w.SyncBlockNum(100 + r, 5000) == 100);
      for (int i = 0; i < 20; ++i) {
        std::string bytes;
        EXPECT(w.RecvBroadcast(&bytes, 5000));
        if (bytes.size() == 64 + static_cast<size_t>(i)) ++got;
      }
      for (int i = 0; i < 100 && !w.shutdown_requested(); ++i) std::this_thread::sleep_for(std::chrono::milliseconds(20));
      EXPECT(w.shutdown_requested());
      w.Stop();
    });
  }
  EXPECT(master.WaitForNodes(5000));
  EXPECT(master.Barrier(5000));
  auto ranges = master.AssignLayers(10, 5000);
  EXPECT(ranges.size() == 3);
  EXPECT(master.SyncBlockNum(100, 5000) == 100);
  for (int i = 0; i < 20; ++i) EXPECT(master.Broadcast(std::string(64 + i, 'x')));
  std::this_thread::sleep_for(std::chrono::milliseconds(200));      // a few heartbeats in both directions
  EXPECT(master.alive() && master.FailedNodes().empty());
  master.ShutdownCluster();
  for (auto& t : workers) t.join();
  master.Stop();
  EXPECT(got.load() == 40);
  std::printf("control plane stress: %d broadcasts received\n", got.load());
}

static void BatchLoopStress() {
  std::atomic<int> pending{0}, done{0}, errors{0};
  BatchLoop loop;
  loop.Start(
      [&]() {
        int p = pending.load();
        while (p > 0 && !pending.compare_exchange_weak(p, p - 1)) {}
        if (p <= 0) return false;
        if (done.fetch_add(1) % 97 == 96) throw std::runtime_error("a failing step");
        return true;
      },
      [&]() { return pending.load() == 0; }, [&](const std::string&) { ++errors; });
  std::vector<std::thread> producers;
  for (int t = 0; t < 4; ++t) {
    producers.emplace_back([&] {
      for (int i = 0; i < 500; ++i) {
        pending.fetch_add(1);
        loop.Notify();
        if (i % 50 == 0) std::this_thread::sleep_for(std::chrono::milliseconds(2));     // let the loop fall asleep
      }
    });
  }
  for (auto& t : producers) t.join();
  for (int i = 0; i < 500 && pending.load() > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(10));
  EXPECT(pending.load() == 0 && done.load() == 2000);
  EXPECT(errors.load() == 2000 / 97);
  loop.Stop();
  EXPECT(!loop.running());
  std::printf("batch loop stress: %d steps, %d errors handled, %lld sleeps\n", done.load(), errors.load(),
              static_cast<long long>(loop.sleeps()));
}

static void WaiterStress() {
  StreamChannel<int> ch;
  Waiter done;
  std::atomic<long long> sum{0};
  std::thread consumer([&] {
    int v = 0, n = 0;
    while (n < 4000) {
      if (ch.Get(&v, 1000)) { sum += v; ++n; }
    }
    done.Set();
  });
  std::vector<std::thread> producers;
  for (int t = 0; t < 4; ++t) producers.emplace_back([&ch] { for (int i = 1; i <= 1000; ++i) ch.Put(i); });
  for (auto& t : producers) t.join();
  EXPECT(done.Wait(10000));
  consumer.join();
  EXPECT(sum.load() == 4LL * 1000 * 1001 / 2 && ch.Size() == 0);
  int v = 0;
  EXPECT(!ch.Get(&v, 10));                       // empty: the time runs out
  std::printf("waiter / channel stress: sum %lld\n", sum.load());
}

static void OtlpStress() {
  OtlpExporter& ex = OtlpExporter::Instance();
  ex.Configure({{"instance", "stress"}}, 200);
  const int64_t dropped0 = ex.dropped();
  std::vector<std::thread> threads;
  for (int t = 0; t < 4; ++t) {
    threads.emplace_back([&ex, t] {
      for (int i = 0; i < 100; ++i) {
        OtlpSpan s;
        s.name = "span"; s.trace_id = std::string(32, 'a'); s.span_id = std::string(16, static_cast<char>('0' + t));
        s.start_us = 1; s.end_us = 2; s.attrs = {{"i", std::to_string(i)}};
        ex.EnqueueSpan("http://127.0.0.1:9/v1/traces", std::move(s));          // the discard port: nobody listens
      }
      ex.EnqueueMetrics("http://127.0.0.1:9/v1/metrics", {{"ksana_x", true, 1, 1.0, 0, 0}}, 1);
    });
  }
  for (auto& t : threads) t.join();
  ex.Flush(10000);
  EXPECT(ex.dropped() > dropped0 && ex.sent() == 0);
  std::printf("otlp stress: %lld requests dropped for an absent collector\n", static_cast<long long>(ex.dropped() - dropped0));
}

int main() {
  SchedulerStress(0);
  SchedulerStress(1);
  SchedulerStress(0, 3);
  SchedulerStress(1, 2);
  ControlPlaneStress();
  BatchLoopStress();
  WaiterStress();
  OtlpStress();
  if (g_failures) {
    std::fprintf(stderr, "%d check(s) failed\n", g_failures);
    return 1;
  }
  std::printf("host stress ok\n");
  return 0;
}
