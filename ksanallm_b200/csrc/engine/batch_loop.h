// The engine's step loop as a native thread (the counterpart of the reference's BatchManager::MainProcess,
// src/ksana_llm/batch_manager/batch_manager.cpp:111-241: schedule, run a step, and sleep on a condition variable when
// there is nothing to run until a request arrives).
//
// The step itself is a callable handed over by the engine (planning is the C++ scheduler, the forward pass is
// launched through PyTorch, so the callable is entered with the interpreter lock held and everything it waits for on
// the GPU releases the lock again). What lives here is the thread, its wake-up and its shutdown: an idle loop costs
// nothing (no polling of the interpreter), `Notify` wakes it within the latency of a condition variable, an
// exception that escapes a step is handed to the error callable and the loop goes on.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <mutex>
#include <string>
#include <thread>

namespace ksana {

class BatchLoop {
 public:
  // step(): runs one engine step, returns whether there was anything to run. idle(): whether the scheduler holds no
  // request at all (then the loop sleeps until notified; otherwise it retries after a millisecond: requests exist but
  // nothing could be scheduled this instant). on_error(message): a step raised.
  using StepFn = std::function<bool()>;
  using IdleFn = std::function<bool()>;
  using ErrorFn = std::function<void(const std::string&)>;

  ~BatchLoop();
  void Start(StepFn step, IdleFn idle, ErrorFn on_error);
  void Notify();                      // a request arrived / was aborted / the engine was told to stop
  void Stop();                        // returns after the thread has ended; safe to call twice
  bool running() const { return running_.load(); }
  int64_t steps() const { return steps_.load(); }
  int64_t sleeps() const { return sleeps_.load(); }

 private:
  void Run();
  StepFn step_;
  IdleFn idle_;
  ErrorFn on_error_;
  std::thread thread_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool notified_ = false;
  std::atomic<bool> stop_{false}, running_{false};
  std::atomic<int64_t> steps_{0}, sleeps_{0};
};

}  // namespace ksana
