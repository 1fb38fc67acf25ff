#include "batch_loop.h"

#include <chrono>
#include <exception>

#include "logger.h"

namespace ksana {

BatchLoop::~BatchLoop() { Stop(); }

void BatchLoop::Start(StepFn step, IdleFn idle, ErrorFn on_error) {
  Stop();
  step_ = std::move(step);
  idle_ = std::move(idle);
  on_error_ = std::move(on_error);
  stop_ = false;
  notified_ = false;
  running_ = true;
  thread_ = std::thread([this]() { Run(); });
}

void BatchLoop::Notify() {
  {
    std::lock_guard<std::mutex> g(mu_);
    notified_ = true;
  }
  cv_.notify_all();
}

void BatchLoop::Stop() {
  stop_ = true;
  Notify();
  if (thread_.joinable()) thread_.join();
  running_ = false;
  step_ = nullptr;
  idle_ = nullptr;
  on_error_ = nullptr;
}

void BatchLoop::Run() {
  KLLM_LOG_DEBUG << "batch loop started";
  while (!stop_) {
    bool ran = false, idle = false;
    try {
      ran = step_();
      if (!ran) idle = idle_();
    } catch (const std::exception& e) {
      KLLM_LOG_ERROR << "engine step failed: " << e.what();
      try {
        if (on_error_) on_error_(e.what());
      } catch (const std::exception& e2) {
        KLLM_LOG_ERROR << "error handler of the batch loop failed: " << e2.what();
      }
    }
    if (ran) {
      ++steps_;
      continue;
    }
    std::unique_lock<std::mutex> lk(mu_);
    if (!notified_ && !stop_) {
      ++sleeps_;
      // nothing at all to do: sleep until a request arrives (with a coarse timeout as a safety net); requests exist
      // but none could run this instant (e.g. all waiting for blocks): look again in a millisecond
      cv_.wait_for(lk, idle ? std::chrono::milliseconds(200) : std::chrono::milliseconds(1), [this]() { return notified_ || stop_.load(); });
    }
    notified_ = false;
  }
  KLLM_LOG_DEBUG << "batch loop ended after " << steps_.load() << " steps";
}

}  // namespace ksana
